"""Version of this package; the reference interface it mirrors is torchsparse 2.1.0."""
__version__ = "0.1.0"
REFERENCE_INTERFACE = "torchsparse 2.1.0"
