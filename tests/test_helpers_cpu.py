"""Host-side helpers that the GPU tests lean on, checked on the CPU: the routing-aware tolerance policy, the sharding of
the oracle's state, the launch-descriptor variants of an LL channel, and the context-parallel threshold policy."""

import torch

from nexrt_b200.config import ShardSpec
from nexrt_b200.models.reference import RefModel, synthetic_prompt
from nexrt_b200.testing import RouteAwareCheck, oracle_state, shard_oracle_state, shrunk_checkpoint


def test_route_aware_check_policy():
    c = RouteAwareCheck([0.1, 0.1, 0.005, 0.1, 0.002, 0.1], tol=2e-2, near=0.01, loose=0.3)
    c.check(0.01, 0)
    c.check(0.019, 1)
    assert c.strict == 2 and not c.flipped
    c.check(0.15, 2)                       # a near tie that did flip
    assert c.flipped
    c.check(0.05, 3)                       # clear-gap token after the flip: 4 x tol
    try:
        c.check(0.09, 3)
        raise SystemExit("a clear-gap token 9 % off must fail even after a flip")
    except AssertionError:
        pass
    c.check(0.2, 4)
    d = RouteAwareCheck([0.1, 0.1])
    try:
        d.check(0.03, 0, 1)                # no near tie in the span: the tight bound applies
        raise SystemExit("must fail")
    except AssertionError:
        pass


def test_shards_of_the_oracle_state_tile_the_whole():
    cfg, ckpt = shrunk_checkpoint(0, cp=True)       # the geometry that also splits four ways
    ref = RefModel(cfg, ckpt)
    ref.prefill(synthetic_prompt(cfg.vocab, 5))
    ref_state = oracle_state(ref)
    for tp in (2, 4):
        parts = [shard_oracle_state(ref_state, cfg, ShardSpec(cfg, tp, r)) for r in range(tp)]
        for idx, whole in ref_state.items():
            if "recurrent_state" in whole:
                assert torch.equal(torch.cat([p[idx]["recurrent_state"] for p in parts]), whole["recurrent_state"])
                D, nqk = cfg.gdn_dim, cfg.gdn_qk_heads
                q = torch.cat([p[idx]["conv_state"][: nqk // tp * D] for p in parts])
                assert torch.equal(q, whole["conv_state"][: nqk * D])
                v = torch.cat([p[idx]["conv_state"][2 * (nqk // tp) * D :] for p in parts])
                assert torch.equal(v, whole["conv_state"][2 * nqk * D :])
            else:
                heads = [p[idx]["k_cache"] for p in parts]
                if tp <= cfg.n_kv_heads:
                    assert torch.equal(torch.cat(heads), whole["k_cache"])
                else:      # ranks of one context-parallel group hold the same kv head
                    assert torch.equal(heads[0], heads[1]) and torch.equal(heads[0], whole["k_cache"][:1])


def test_channel_variants_share_the_inbox():
    from nexrt_b200.parallel.channel import LLChannel

    ch = LLChannel(torch.device("cpu"), 1, 0, 64)
    v = ch.variant(multicast=False, budget_ms=50)
    assert v.local == ch.struct.local and v.seq == ch.struct.seq and v.status == ch.struct.status
    assert v.budget_ns == 50_000_000 and ch.struct.budget_ns != v.budget_ns and not v.mc
    v.world = 7
    assert ch.struct.world == 1            # a copy, not a view


def test_cp_threshold_depends_on_the_group_size(monkeypatch):
    import nexrt_b200.decode_engine as de

    class Fake:
        cp_threshold = de.DecodeEngine.cp_threshold

    monkeypatch.delenv("NEXRT_CP_THRESHOLD", raising=False)
    cfg, _ = shrunk_checkpoint(0)
    f = Fake()
    f.spec = type("S", (), {"cp_size": 2})()
    assert f.cp_threshold == 1 << 30                      # groups of two never win: off unless asked for
    f.spec = type("S", (), {"cp_size": 4})()
    assert f.cp_threshold == de.CP_THRESHOLD == 96 * 1024
    monkeypatch.setenv("NEXRT_CP_THRESHOLD", "1000")
    f.spec = type("S", (), {"cp_size": 2})()
    assert f.cp_threshold == de.CP_THRESHOLD              # an explicit setting applies to every group size


def test_host_side_modules_import_without_torch_from_any_directory(tmp_path):
    """The serving front ends, the cache / consensus / supervisor logic, the protocol model and the build helper are plain
    Python: importing them from outside the repository must neither need the working directory nor pull in torch
    (a front-end box has no GPU stack).  The heavier packages then import too.  Reference: tests/test_package_imports.py."""
    import os
    import subprocess
    import sys
    from pathlib import Path

    light = ("nexrt_b200", "nexrt_b200.serve", "nexrt_b200.parallel", "nexrt_b200.runtime", "nexrt_b200.utils", "nexrt_b200.build",
             "nexrt_b200.config", "nexrt_b200.sampling", "nexrt_b200.runtime.control", "nexrt_b200.runtime.rounds", "nexrt_b200.parallel.ll_model",
             "nexrt_b200.serve.cache_lifecycle", "nexrt_b200.serve.cache_consensus", "nexrt_b200.serve.serve_control",
             "nexrt_b200.serve.process_supervisor", "nexrt_b200.serve.stream_protocol", "nexrt_b200.serve.bridge_client",
             "nexrt_b200.serve.stream_chat", "nexrt_b200.serve.openai_serve", "nexrt_b200.serve.launch")
    heavy = ("nexrt_b200.dflash.config", "nexrt_b200.mtp.reference", "nexrt_b200.weights", "nexrt_b200.decode_engine", "nexrt_b200.serve.bridge_serve")
    repo = Path(__file__).resolve().parents[1]
    assert repo not in (tmp_path, *tmp_path.parents)
    script = "\n".join((
        "import importlib, sys",
        f"light, heavy = {light!r}, {heavy!r}",
        "for m in light:",
        "    importlib.import_module(m)",
        "    assert 'torch' not in sys.modules, m",
        "for m in heavy:",
        "    importlib.import_module(m)",
        "print('ok')",
    ))
    env = dict(os.environ, PYTHONPATH=str(repo), PYTHONDONTWRITEBYTECODE="1")
    done = subprocess.run([sys.executable, "-c", script], cwd=tmp_path, env=env, text=True, capture_output=True, check=False, timeout=300)
    assert done.returncode == 0 and done.stdout.strip() == "ok", done.stderr[-2000:]


def test_no_library_collective_on_the_step_path():
    """Every all-reduce / exchange of a step happens inside the step's own kernels; the block wrappers and the
    speculative blocks never call a torch.distributed collective (reference tests/test_dflash_static.py:
    test_public_kernel_surface, the runtime block holds no collective).  The one library call that exists is the
    explicitly selected baseline arm of the context (``collective == "nccl"``)."""
    from pathlib import Path

    root = Path(__file__).resolve().parents[1] / "nexrt_b200"
    step_path = ["gdn.py", "attn.py", "moe.py", "head.py", "ctl_mirror.py", "prefill_wide.py", "m4_verify.py", "m8_verify.py",
                 "mtp/block.py", "dflash/block.py", "ops/wide.py", "ops/tc_gemm.py", "runtime/rounds.py"]
    calls = ("all_reduce(", "all_gather(", "reduce_scatter(", "all_to_all(", "broadcast(")      # (host barriers exist in the reset paths between steps)
    for name in step_path:
        text = (root / name).read_text(encoding="utf-8")
        for call in calls:
            assert call not in text, (name, call)
    ctx = (root / "runtime/context.py").read_text(encoding="utf-8")
    assert ctx.count("dist.all_reduce(") == 1 and 'if self.collective != "nccl":\n            return' in ctx


def test_packaging_metadata_names_real_entry_points():
    """pyproject.toml: every console script resolves to a callable of the package, the package data covers the CUDA
    sources the in-place build needs, and the gpu marker stays registered by conftest (no second registry)."""
    import importlib
    import tomllib
    from pathlib import Path

    root = Path(__file__).resolve().parents[1]
    meta = tomllib.loads((root / "pyproject.toml").read_text(encoding="utf-8"))
    scripts = meta["project"]["scripts"]
    assert {"nexrt-serve", "nexrt-openai", "nexrt-client", "nexrt-build", "nexrt-extract-layers"} <= set(scripts)
    for name, target in scripts.items():
        module, func = target.split(":")
        assert callable(getattr(importlib.import_module(module), func)), name
    patterns = meta["tool"]["setuptools"]["package-data"]["nexrt_b200"]
    csrc = root / "nexrt_b200" / "csrc"
    covered = {p.name for pat in patterns for p in (root / "nexrt_b200").glob(pat)}
    assert {p.name for p in csrc.iterdir() if p.suffix in (".cu", ".cuh", ".h")} <= covered


def test_bench_clock_sampler_against_a_fake_nvml(monkeypatch):
    """``bench.NvmlClocks`` only READS: SM clock, maximum clock and throttle reasons.  With a fake ``pynvml`` the summary is
    the median clock, the named reasons that were active in any sample, and at least the two samples taken at the
    start and the end of the region; without NVML it reports no samples rather than failing the benchmark."""
    import sys
    import time
    import types
    from pathlib import Path

    sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
    import bench

    fake = types.ModuleType("pynvml")
    fake.NVML_CLOCK_SM = 1
    fake.nvmlClocksThrottleReasonHwSlowdown, fake.nvmlClocksThrottleReasonSwPowerCap = 0x8, 0x4
    fake.nvmlClocksThrottleReasonHwThermalSlowdown, fake.nvmlClocksThrottleReasonSwThermalSlowdown = 0x40, 0x20
    calls = {"n": 0, "writes": 0}
    clocks = [1965, 1965, 1310, 1965, 1965]
    fake.nvmlInit = lambda: None
    fake.nvmlDeviceGetHandleByIndex = lambda i: ("gpu", i)
    fake.nvmlDeviceGetMaxClockInfo = lambda h, kind: 1965

    def clock(h, kind):
        calls["n"] += 1
        return clocks[min(calls["n"] - 1, len(clocks) - 1)]

    fake.nvmlDeviceGetClockInfo = clock
    fake.nvmlDeviceGetCurrentClocksThrottleReasons = lambda h: 0x4 if calls["n"] == 3 else 0
    for setter in ("nvmlDeviceSetApplicationsClocks", "nvmlDeviceSetGpuLockedClocks", "nvmlDeviceResetGpuLockedClocks", "nvmlDeviceSetPowerManagementLimit"):
        setattr(fake, setter, lambda *a, **k: calls.__setitem__("writes", calls["writes"] + 1))
    monkeypatch.setitem(sys.modules, "pynvml", fake)
    s = bench.NvmlClocks(0, period_s=0.002).start()
    time.sleep(0.05)
    out = s.stop()
    assert out["sm_max_mhz"] == 1965.0 and out["sm_mhz"] == 1965.0 and out["samples"] >= 3 and out["reasons"] == ["sw_power_cap"]
    assert calls["writes"] == 0                       # nothing that changes a GPU setting was called
    broken = types.ModuleType("pynvml")
    broken.nvmlInit = lambda: (_ for _ in ()).throw(RuntimeError("no driver"))
    monkeypatch.setitem(sys.modules, "pynvml", broken)
    assert bench.NvmlClocks(0).start().stop() == {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}


def test_reference_arm_reports_one_unavailable_line_and_exits_zero():
    """``bench.py --impl reference`` where the reference cannot run: exactly one JSON line with ``impl`` and a one-line
    reason, exit code 0."""
    import json
    import subprocess
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parents[1]
    done = subprocess.run([sys.executable, str(root / "bench.py"), "--impl", "reference"], capture_output=True, text=True, timeout=300, cwd=root)
    lines = [l for l in done.stdout.splitlines() if l.strip()]
    assert done.returncode == 0 and len(lines) == 1, (done.returncode, done.stdout[-500:], done.stderr[-500:])
    rec = json.loads(lines[0])
    assert rec["impl"] == "reference" and isinstance(rec["unavailable"], str) and rec["unavailable"] and "\n" not in rec["unavailable"]
