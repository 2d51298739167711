"""gTop-k S-SGD trainer command line under the reference's module name; start
one process per GPU with torchrun (see gtopk_run.sh)."""
from gtopkssgd_b200.trainer.gtopk_trainer import build_parser, main, robust_ssgd  # noqa: F401

if __name__ == "__main__":
    main()
