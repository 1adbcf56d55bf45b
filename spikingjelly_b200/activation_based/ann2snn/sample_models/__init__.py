from . import cifar10_resnet, mnist_cnn  # noqa: F401
