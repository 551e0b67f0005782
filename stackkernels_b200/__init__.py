"""B200-native attention hot path (flash_attention fwd/bwd, flash_decode) behind the
StackKernels PyTorch API.  Compute lives in ``libskb200.so`` (hand-written CUDA, sm_100a)."""
from ._options import get_backend, options, set_backend
from .attention import FlashAttention, FlashAttentionFunction, flash_attention, flash_decode
from .embedding import RoPE, RoPEFunction, apply_rope, kv_cache_append, precompute_freqs
from .host import flash_attention_host
from .launchers import flash_decode_paged
from .varlen import FlashAttentionVarlenFunction, flash_attention_varlen

__all__ = ["flash_attention", "flash_attention_varlen", "FlashAttentionVarlenFunction", "flash_decode",
           "flash_decode_paged", "flash_attention_host", "apply_rope", "RoPE", "RoPEFunction",
           "precompute_freqs", "kv_cache_append", "FlashAttention", "FlashAttentionFunction",
           "get_backend", "set_backend", "options"]
__version__ = "0.1.0"
