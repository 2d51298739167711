"""``MnistNet`` under the reference's module name."""
from gtopkssgd_b200.models.mnistnet import MnistNet  # noqa: F401


def model_builder(dnn="mnistnet", num_classes=10, **kwargs):
    from gtopkssgd_b200.models import create_net
    return create_net(num_classes, dnn, **kwargs)[0]
