"""Entry-point package: ``python -m train.train_qwen --config X.toml [--section.key value ...]``
(the same command line as the reference, reference: scripts/finetune.sh:14-18)."""
