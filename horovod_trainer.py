"""The reference's dense entry point name.  Horovod is not used: the dense
all-reduce runs on NCCL through torch.distributed (dense_trainer.py)."""
from gtopkssgd_b200.trainer.dense_trainer import main, ssgd_dense, ssgd_with_horovod  # noqa: F401

if __name__ == "__main__":
    main()
