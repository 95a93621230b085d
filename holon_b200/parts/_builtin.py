"""Registers the parts that ship with the framework."""
from .attention import GQA
from .base import register_part
from .block import PreNorm
from .embedding import Embedding, Head
from .feedforward import SwiGLU
from .norm import RMSNorm
from .position import Rope

register_part("norm", "rmsnorm", RMSNorm, replace=True)
register_part("position", "rope", Rope, replace=True)
register_part("mixer", "gqa", GQA, replace=True)
register_part("ffn", "swiglu", SwiGLU, replace=True)
register_part("block", "prenorm", PreNorm, replace=True)
register_part("embed", "table", Embedding, replace=True)
register_part("head", "linear", Head, replace=True)
