"""B200-native (sm_100a) replacement for the attention hot path of niw/mmh3's diffusion transformer.

The product is `lib/libmmh3_attn_b200.so`, a C-ABI library (see include/mmh3_attention.h). This
package builds it (`mmh3_b200.build`) and mirrors the reference's host-side wrappers over it
(`mmh3_b200.attention`, `mmh3_b200.vsa`, `mmh3_b200.shard`).
"""

__all__ = ["attention", "vsa", "shard", "synthetic", "build"]
