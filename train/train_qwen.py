"""``torchrun ... -m train.train_qwen --config configs/<x>.toml [--training.tp_size 2 ...]``."""
from vlm_training_b200.train.trainer import Trainer, main  # noqa: F401

if __name__ == "__main__":
    main()
