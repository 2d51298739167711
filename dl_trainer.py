"""Single-GPU trainer command line and the ``DLTrainer`` class under the
reference's module name.  ``python dl_trainer.py --dnn resnet20 --dataset cifar10 --data-dir synthetic``"""
from gtopkssgd_b200.trainer.dl_trainer import (DLTrainer, _support_datasets, _support_dnns, create_net,  # noqa: F401
                                                main, train_with_single)

if __name__ == "__main__":
    main()
