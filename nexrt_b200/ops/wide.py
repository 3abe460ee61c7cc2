"""Launch helpers of the wide (multi-row) projections that several blocks share."""

from __future__ import annotations

from .lib import check, ptr


def oproj_allreduce(c, inp, z, gnorm_w, w, w_s, K: int, M: int, mode: int, hd: int, cp_ref, cp_site: int) -> None:
    """Out-projection + tensor-parallel all-reduce + residual for M >= ``c.tc_oproj_rows`` rows: a staging kernel builds
    the input rows (plain / gated norm / context-parallel merge) as e4m3 planes, then one tcgen05 GEMM streams the
    weights once for all rows and all-reduces in its epilogue (csrc/oproj.cu, csrc/tc_moe.cu)."""
    lib, st, cfg = c.lib, c.stream(), c.cfg
    check(lib.nexrt_oproj_stage_split(ptr(inp), ptr(z), ptr(gnorm_w), ptr(c.oproj_planes), ptr(c.oproj_descale), K, M, mode, cfg.rms_eps, hd, cp_ref,
                                      cp_site, st), "oproj_stage_split")
    check(lib.nexrt_tc_oproj_allreduce(ptr(c.oproj_planes), ptr(c.oproj_descale), ptr(w), ptr(w_s), ptr(c.x), ptr(c.zero_ids), cfg.hidden, K, M, 0,
                                       c.channel.ref, c.next_site(), ptr(c.status), st), "tc_oproj_allreduce")


def oproj_is_wide(c, K: int, M: int) -> bool:
    return M >= c.tc_oproj_rows and c.cfg.hidden % 128 == 0 and K % 128 == 0 and K <= 8192
