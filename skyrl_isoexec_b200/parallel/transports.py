"""One call that gives every parallel group of a job its peer-memory transport (when the GPUs can reach each other):

  data parallel    ``SymmGroup``  gradient sum over symmetric memory              (csrc/peer_collectives.cu)
  tensor parallel  ``FusedTP``    GEMM fused with all-reduce / reduce-scatter / all-gather (csrc/tp_gemm_fused.cu)
  expert parallel  ``EPPeer``     dispatch, grouped expert GEMMs and row return   (csrc/moe_ep_peer.cu, moe_grouped_gemm.cu)

Without peer access (or on CPU) nothing is registered and every path uses its NCCL / gloo transport.
"""

from __future__ import annotations

import torch

from . import nccl_runtime


def setup_transports(ps, model_cfg=None, max_tokens: int = 8192, dp_staging_bytes: int = 512 << 20) -> dict:
    """Collective: every rank of the job calls it with the same arguments. Returns what was registered."""
    out = {"dp": False, "tp": False, "ep": False}
    if not torch.cuda.is_available():
        return out
    caps = nccl_runtime.capabilities()
    if not caps["symmetric_memory"]:
        return out
    import os

    if os.environ.get("SKYRL_ISOEXEC_PIK_P2P", "1") == "0":
        return out          # forced onto the NCCL all-gather transport of the tree reductions (same bits, other wire)
    if ps.dp > 1 and ps.dp & (ps.dp - 1) == 0 and ps.dp <= 16:
        from .symm_runtime import SymmGroup

        SymmGroup(ps.dp_group, staging_bytes=dp_staging_bytes)
        out["dp"] = True
    if ps.tp > 1 and ps.tp in (2, 4, 8) and model_cfg is not None:
        from . import tp_fused

        h = model_cfg.hidden_size
        stage = max_tokens * h * 4 + (1 << 20)                     # fp32 partial of one [tokens, hidden] output per half
        k_max = max(h, model_cfg.ffn_size // ps.tp, model_cfg.num_q_heads * model_cfg.head_dim // ps.tp)
        tp_fused.register(ps.tp_group, tp_fused.FusedTP(ps.tp_group, stage_bytes=stage, out_bytes=max_tokens * h * 2 + (1 << 20),
                                                        gather_bytes=max_tokens * k_max * 2 + (1 << 20)))
        out["tp"] = True
    if ps.ep > 1 and model_cfg is not None and model_cfg.has_moe and model_cfg.num_experts % ps.ep == 0:
        from ..ops import moe_ep

        rows = max_tokens * model_cfg.top_k
        moe_ep.register(ps.ep_group, moe_ep.EPPeer(ps.ep_group, model_cfg.hidden_size, model_cfg.num_experts, max_rows_local=rows,
                                                    capacity_rows=min(rows * ps.ep, rows * 4)))
        out["ep"] = True
    return out
