"""Which libraries exist and with which compile-time sizes they can be asked for."""

from __future__ import annotations

from .build import LIBRARIES


def all_build_requests():
    """(name, sources, defines, extra headers) of everything worth pre-building."""
    reqs = [("core", LIBRARIES["core"], {}, [])]
    reqs.append(("stream", ["gemm_stream.cu", "gemm_stream_tma.cu"], {}, []))
    reqs.append(("tcgen05", ["gemm_tcgen05.cu"], {}, []))
    reqs.append(("attn_tcgen05", ["attention_tcgen05.cu"], {}, []))
    for hd in (64, 128):
        reqs.append((f"attn_mma_hd{hd}", ["attention_mma.cu"], {"IE_HD": hd}, ["attention_noalloc.h"]))
        reqs.append((f"attn_mma_hd{hd}_bias", ["attention_mma.cu"], {"IE_HD": hd, "IE_ATTN_BIAS": 1}, ["attention_noalloc.h"]))
    for dk, dv in ((64, 64), (64, 128), (128, 128)):   # (key, value) head sizes of the float32-score attention worth having early
        reqs.append((f"attn_wide_k{dk}_v{dv}", ["attention_wide.cu"], {"IE_AW_DK": dk, "IE_AW_DV": dv}, []))
    for d in (16, 24, 32, 48, 64, 128):  # head sizes of the delta-rule mixer worth having before a model asks
        reqs.append((f"delta_rule_d{d}", ["delta_rule.cu"], {"IE_DR_DIM": d}, []))
    for dk, dv in ((64, 64), (64, 128), (128, 128)):   # (key, value) head sizes of the gated delta rule worth having early
        reqs.append((f"gated_delta_k{dk}_v{dv}", ["gated_delta.cu"], {"IE_GD_DK": dk, "IE_GD_DV": dv}, []))
    return reqs
