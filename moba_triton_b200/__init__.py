from moba_triton_b200.config import MoBAConfig
__all__ = ["MoBAConfig"]
