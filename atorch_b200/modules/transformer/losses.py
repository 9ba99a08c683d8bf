from .cross_entropy import AtorchCrossEntropyLoss, CrossEntropyLoss  # noqa: F401
