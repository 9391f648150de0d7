"""Module-level switch of the causal-local f16 dQ pre-scale, at the name the reference's callers use
(flash_attn/cute/interface_bwd_fp4.py:938 DQ_CAUSAL_PRESCALE, default False; README.md:56-61 of the reference).

False: one power-of-two pre-scale per batch row / document. True (batched causal s_q == s_k): one per query tile, sized
from that tile's own dO rows and the PREFIX of key tiles it may see, so a later key cannot move an earlier query's dQ
rounding. Read by the plan when a call is resolved; the resolved value travels in the plan.
"""
DQ_CAUSAL_PRESCALE = False

# With DQ_CAUSAL_PRESCALE on: "tile" = one pre-scale per 128-query tile (the reference's form on its CTA-pair backward),
# "row" = one per query row from per-token statistics and running maxima over the keys j <= i (the reference's form on its
# 1-CTA backward, flash_attn/cute/interface_bwd_fp4.py:1007-1012 "rowwise": exactly causal, no key-tile granularity).
DQ_CAUSAL_GRANULARITY = "tile"
