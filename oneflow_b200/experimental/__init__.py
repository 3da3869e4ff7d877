from .load_mnist import load_mnist  # noqa: F401
