"""Per-engine launch context: control block, residual rows, LL channel, scratch and site counting.

The reference allocates these per block object and wires them together in
``DecodeEngine.__init__`` (``nex_n2_5_pro/decode_engine.py:87-202``); here one context owns the
buffers every block of an engine shares, so a 60-layer stack carries one set of scratch.
"""

from __future__ import annotations

import os

import torch

from ..config import ModelConfig, ShardSpec
from ..ops import lib as L
from ..parallel.channel import LLChannel
from .audit import guarded_zeros, violated
from .control import CTL_WORDS, Ctl

MAX_ROWS = 8
MAX_TOPK = 28


class StepContext:
    def __init__(self, cfg: ModelConfig, spec: ShardSpec, device: torch.device, group=None, budget_ms=None, cp: bool = False,
                 comm_world=None, comm_rank=None, collective: str = "fused"):
        self.cfg, self.spec, self.device, self.group = cfg, spec, device, group
        self.lib = L.load()
        self.tp, self.rank = spec.tp, spec.rank
        # shapes may be those of one rank of a wider group while running alone (profiling fixture)
        cw = spec.tp if comm_world is None else comm_world
        cr = spec.rank if comm_rank is None else comm_rank
        props = torch.cuda.get_device_properties(device)
        self.n_cta = props.multi_processor_count
        H = cfg.hidden
        i32, f32, bf = torch.int32, torch.float32, torch.bfloat16
        # NEXRT_CANARY=1: every scratch buffer gets guard bands (runtime/audit.py) that ``canaries_violated`` checks
        self._guards = [] if os.environ.get("NEXRT_CANARY", "0") == "1" else None

        def z(*shape, dtype=f32):
            if self._guards is None:
                return torch.zeros(*shape, dtype=dtype, device=device)
            return guarded_zeros(self._guards, shape, dtype, device)

        self.ctl = z(CTL_WORDS, dtype=i32)
        self.ctl[Ctl.EOS] = -1
        self.ctl[Ctl.STOP_POS] = -1
        self.x = z(MAX_ROWS, H, dtype=bf)
        self.seq = torch.ones(1, dtype=i32, device=device)
        self.status = self.ctl[Ctl.STATUS : Ctl.STATUS + 1]
        kw = {} if budget_ms is None else {"budget_ms": budget_ms}
        self.channel = LLChannel(device, cw, cr, MAX_ROWS * H, group=group, seq=self.seq, status=self.status, **kw)
        # Library-baseline arm (collective="nccl"): the projection kernels that normally end in the in-kernel all-reduce
        # store their fp32 partial sums instead, and an NCCL all-reduce plus a residual-add kernel follow as separate
        # graph nodes - the arm the fused epilogues are measured against.  One-row steps only.
        self.collective = collective
        self.ar_channel = self.channel
        self.ar_partial = None
        if collective == "nccl":
            self.ar_channel = LLChannel(device, 1, 0, MAX_ROWS * H, group=None, seq=self.seq, status=self.status, **kw)
            self.ar_partial = z(MAX_ROWS, H)
            self.lib.nexrt_set_partial_out(self.ar_partial.data_ptr())
        elif collective != "fused":
            raise ValueError(f"unknown collective arm {collective!r}")
        self.cp_channel = None
        if cp and spec.cp_size > 1 and cw == spec.tp:
            slots = MAX_ROWS * spec.q_heads * (cfg.head_dim + 1)
            self.cp_channel = LLChannel(
                device, spec.tp, spec.rank, slots, group=group, seq=self.seq, status=self.status, members=spec.cp_group, **kw
            )
        # gated delta net scratch
        self.gdn_qkv = z(MAX_ROWS, max(spec.gdn_qkv_rows, 1))
        self.gdn_z = z(MAX_ROWS, max(spec.gdn_local, 1))
        self.gdn_beta = z(MAX_ROWS, max(spec.gdn_v, 1))
        self.gdn_g = z(MAX_ROWS, max(spec.gdn_v, 1))
        self.gdn_out = z(MAX_ROWS, max(spec.gdn_local, 1))
        # attention scratch (sized for the context-parallel front: every q head of the kv group)
        hd = cfg.head_dim
        nq_max = spec.q_heads * (spec.cp_size if cp else 1)
        self.q_raw = z(MAX_ROWS, nq_max, hd)
        self.gate = z(MAX_ROWS, spec.q_heads, hd)
        self.k_raw = z(MAX_ROWS, spec.kv_heads, hd)
        self.attn_out = z(MAX_ROWS, spec.q_heads * hd)
        self.n_splits = max(1, self.n_cta // spec.kv_heads)
        rows_max = MAX_ROWS * (nq_max // spec.kv_heads)
        self.ws_acc = z(spec.kv_heads, self.n_splits, rows_max, hd)
        self.ws_ml = z(spec.kv_heads, self.n_splits, rows_max, 2)
        self.attn_ticket = z(spec.kv_heads, dtype=i32)
        half = cfg.rotary_dim // 2
        self.inv_freq = (1.0 / (cfg.rope_theta ** (torch.arange(0, cfg.rotary_dim, 2, dtype=f32) / cfg.rotary_dim))).to(device)
        assert self.inv_freq.numel() == half
        # mixture of experts scratch
        S = cfg.top_k + 1
        self.moe_logits = z(MAX_ROWS, cfg.n_experts + 1)
        self.moe_ids = z(MAX_ROWS, S, dtype=i32)
        self.moe_wts = z(MAX_ROWS, S)
        self.moe_gu = z(MAX_ROWS, S, 2 * spec.inter)
        self.moe_ticket = z(1, dtype=i32)
        self.moe_partial = z(4, MAX_ROWS, (cfg.n_experts + 1 + 15) // 16 * 16)
        # scratch of the tcgen05 expert kernels (multi-row steps): e4m3 activation planes and per-row scales
        self.moe_planes1 = z(3 * MAX_ROWS, cfg.hidden, dtype=torch.uint8)
        self.moe_planes2 = z(3 * MAX_ROWS, S * spec.inter, dtype=torch.uint8)
        self.moe_descale = z(MAX_ROWS)
        self.moe_ksplit = int(os.environ.get("NEXRT_MOE_KSPLIT", "2"))              # K-split of the tcgen05 gate/up product
        self.moe_gu_tc = z(self.moe_ksplit, MAX_ROWS, S, 2 * spec.inter)          # its partial planes
        self.wide_xn = z(MAX_ROWS, cfg.hidden)                                    # fp32 normalised rows (b/a rows of the wide GDN front)
        self.wide_ksplit = int(os.environ.get("NEXRT_WIDE_KSPLIT", "4"))                                                       # K-split of the wide front GEMMs (partials summed by the tail)
        cp_front_rows = (spec.q_heads * spec.cp_size + spec.q_heads + 2 * spec.kv_heads) * cfg.head_dim
        self.wide_pre = z(self.wide_ksplit, MAX_ROWS, max(spec.gdn_front_rows, spec.attn_front_rows, cp_front_rows))  # projections of the wide fronts
        self.zero_ids = z(MAX_ROWS, dtype=torch.int32)
        self.oproj_planes = z(3 * MAX_ROWS, max(spec.gdn_local, spec.attn_local), dtype=torch.uint8)
        self.oproj_descale = z(MAX_ROWS)
        self.tc_oproj_rows = int(os.environ.get("NEXRT_TC_OPROJ_ROWS", "0")) or 1 << 30   # measured no faster than the fused kernel at 4 and 8 rows: off unless asked for
        self.router_ksplit = 8
        self.router_planes = z(2 * MAX_ROWS, cfg.hidden, dtype=torch.bfloat16)
        self.router_partial = z(self.router_ksplit, MAX_ROWS, (cfg.n_experts + 1 + 15) // 16 * 16)
        # head scratch
        self.head_cand = z(MAX_ROWS, self.n_cta, MAX_TOPK, dtype=torch.int64)
        self.head_ticket = z(1, dtype=i32)
        self.head_export = z(MAX_ROWS, 64, dtype=i32)
        self.sampling = z(8, dtype=torch.int64)
        self.site = 0
        self._rope = {}
        self.early_ctl = os.environ.get("NEXRT_EARLY_CTL", "1") != "0"

    def canaries_violated(self):
        """Names of the scratch buffers whose guard bands were written (``NEXRT_CANARY=1`` only; ``None`` when off)."""
        if self._guards is None:
            return None
        torch.cuda.synchronize(self.device)
        bad = violated(self._guards)
        if not bad:
            return []
        by_ptr = {t.data_ptr(): name for name, t in vars(self).items() if isinstance(t, torch.Tensor)}
        return [by_ptr.get(self._guards[i][0].data_ptr() + 256, f"allocation {i}") for i in bad]

    def rope_table(self, cache_len: int) -> torch.Tensor:
        """(cos, sin) of position * inv_freq for every cache position, built once per engine like the
        reference's RoPE tables (``nex_n2_5_pro/attn.py:171-177``)."""
        t = self._rope.get(cache_len)
        if t is None:
            ang = torch.arange(cache_len, dtype=torch.float32, device=self.device)[:, None] * self.inv_freq[None, :]
            t = torch.stack([torch.cos(ang), torch.sin(ang)], -1).contiguous()
            self._rope[cache_len] = t
        return t

    # ---- site counting: one index per launch that touches an LL channel -----------------------
    def begin_step(self) -> None:
        self.site = 0

    def next_site(self) -> int:
        s = self.site
        self.site += 1
        return s

    def stream(self) -> int:
        return torch.cuda.current_stream(self.device).cuda_stream

    def after_allreduce(self, M: int) -> None:
        """Library-baseline arm: sum the partial rows the last projection kernel stored over the ranks with NCCL, then add
        them to the residual rows (two more graph nodes per site).  Nothing to do in the fused arm."""
        if self.collective != "nccl":
            return
        import torch.distributed as dist

        if self.tp > 1 and dist.is_initialized():
            dist.all_reduce(self.ar_partial[:M], group=self.group)
        L.check(self.lib.nexrt_residual_add(self.x.data_ptr(), self.ar_partial.data_ptr(), M * self.cfg.hidden, self.stream()), "residual_add")
