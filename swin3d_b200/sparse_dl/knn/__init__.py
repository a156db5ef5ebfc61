from .knn import KNN  # noqa: F401

__all__ = ["KNN"]
