"""Checkpoint evaluator under the reference's module name."""
from gtopkssgd_b200.trainer.evaluate import evaluate, main, model_average, parse_model_dir  # noqa: F401

if __name__ == "__main__":
    main()
