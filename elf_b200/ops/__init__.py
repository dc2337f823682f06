"""Hand-written sm_100a kernels and their Python entry points.

``elf_b200.ops.gemm``      tcgen05/TMEM GEMM family: forward, input-grad, weight-grad (+accumulate)
``elf_b200.ops.fused``     RMSNorm, RoPE, SwiGLU, cross-entropy, embedding, AdamW (bandwidth-bound kernels)
``elf_b200.ops.attention`` causal GQA flash attention forward/backward

The compiled extension lives next to the sources (``elf_b200/csrc``) and is built by
``python -m elf_b200.csrc.build`` (or ``__graft_entry__.build()``).  On a machine with a
GPU the ops raise if the extension is missing instead of silently using torch.
"""

from . import _ext  # noqa: F401
