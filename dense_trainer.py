"""Dense (NCCL all-reduce) S-SGD trainer command line; see dense_run.sh."""
from gtopkssgd_b200.trainer.dense_trainer import main, ssgd_dense, ssgd_with_horovod  # noqa: F401

if __name__ == "__main__":
    main()
