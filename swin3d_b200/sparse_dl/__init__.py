"""Drop-in counterpart of the reference package Swin3D.sparse_dl (autograd Functions)."""
