from .knn import KNN  # noqa: F401
from .consumers import (KNNInterpolate, KNNMaxPool, get_offset, knn_linear_interpolation,  # noqa: F401
                        knn_max_pool, query_knn_feature)

__all__ = ["KNN", "KNNInterpolate", "KNNMaxPool", "get_offset", "knn_linear_interpolation",
           "knn_max_pool", "query_knn_feature"]
