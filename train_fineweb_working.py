"""HF-Trainer variant on Dolma-style streaming data (counterpart of the reference's
``scripts/train_hf.py`` and ``train_fineweb_working.py``): same flags as ``train_production.py``."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


from train_production import MoEModelWrapper, load_config, main  # noqa: E402,F401


def __getattr__(name):          # the Trainer subclasses are built on first use (they need transformers)
    import train_production
    return getattr(train_production, "MoETrainer" if name == "MuonTrainer" else name)


SimpleModelWrapper = MoEModelWrapper          # the names this variant of the script uses for the same two classes


def tokenize_function(examples, tokenizer=None, max_length: int = 2048):
    """Tokenise a batch of ``{"text": [...]}`` rows, truncated to ``max_length``, no padding."""
    if tokenizer is None:
        raise ValueError("pass the tokenizer: tokenize_function(examples, tokenizer, max_length)")
    return tokenizer(examples["text"], truncation=True, max_length=max_length, padding=False)


if __name__ == "__main__":
    main()
