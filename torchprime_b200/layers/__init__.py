from .sequential import HomogeneousSequential

__all__ = ["HomogeneousSequential"]
