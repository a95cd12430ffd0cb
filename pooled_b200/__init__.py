"""pooled_b200: pooled's GQA attention hot path on B200.

The product is libpooled_attn.so (CUDA for sm_100a behind the C ABI of include/pooled_attn.h).  This package
is the host side above it: `lib` binds the C ABI with ctypes, `attn` mirrors the attention call surface of
pooled's engines (engine/qwen35.js _encodeLayerR / _encAttnCore, engine/wgsl/attn_dec.js host mirrors) and
`shard` runs the KV-sequence-sharded decode over torch.distributed.  There is no CPU path: importing works
without a GPU, every compute call needs the CUDA library and a B200.
"""
from .lib import PA_F16, PA_F32, PaError, Lib, load  # noqa: F401
from .attn import (AttnConfig, AttnEngine, DEC_CQ, attn_dec_config, attn_tile_config, dec_split_len, dec_splits,  # noqa: F401
                   tile_split_len)
