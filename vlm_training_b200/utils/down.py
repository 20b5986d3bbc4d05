"""Download an HF snapshot: ``python -m vlm_training_b200.utils.down <repo_id> [local_dir]``
(reference: utils/down.py:1-6)."""
import sys


def main(argv=None):
    argv = sys.argv[1:] if argv is None else argv
    if not argv:
        raise SystemExit("usage: python -m vlm_training_b200.utils.down <repo_id> [local_dir]")
    from huggingface_hub import snapshot_download

    print(snapshot_download(repo_id=argv[0], local_dir=argv[1] if len(argv) > 1 else None))


if __name__ == "__main__":
    main()
