from .attn_coff import (SelfAttnAIOFunction, PosEmb, TableDims, IndexMode,  # noqa: F401
                        PrecisionMode)
