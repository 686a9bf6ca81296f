"""HF-Trainer variant on Dolma-style streaming data (counterpart of the reference's
``scripts/train_hf.py`` and ``train_fineweb_working.py``): same flags as ``train_production.py``."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


from train_production import MoEModelWrapper, load_config, main  # noqa: E402,F401


def __getattr__(name):          # MoETrainer, TrueLossLoggingCallback: built on first use (they need transformers)
    import train_production
    return getattr(train_production, name)


if __name__ == "__main__":
    main()
