"""Tensor-parallel engine on 2 GPUs as child processes (torchrun, NCCL bootstrap, in-kernel LL
all-reduce over symmetric memory), with NVSwitch multicast and with plain peer stores."""

import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _run(world, env_extra, port, script="tp_worker.py"):
    env = dict(os.environ, **env_extra)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(HERE, script)]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    if r.returncode != 0:
        # the ranks' own tracebacks sit above torchrun's summary: keep the lines that name the failure
        keep = [ln for ln in (r.stdout + "\n" + r.stderr).splitlines() if any(k in ln for k in ("Error", "assert", "File \"", "rank"))]
        r.stderr = "\n".join(keep[:60]) + "\n...\n" + r.stderr[-1500:]
    return r


@pytest.mark.parametrize("mode", ["auto", "peer-stores"])
def test_tp2_matches_oracle(mode):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    extra = {"NEXRT_WAIT_BUDGET_MS": "5000"}
    if mode == "peer-stores":
        extra.update(NEXRT_NO_MULTICAST="1", NCCL_NVLS_ENABLE="0")
    r = _run(2, extra, 29611 if mode == "auto" else 29612)
    assert r.returncode == 0 and "TP_WORKER_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


def test_context_parallel_tp4():
    """4 ranks, 2 kv heads: context-parallel groups of 2 (partial exchange + LSE merge in the
    out-projection prologue) against the oracle."""
    if torch.cuda.device_count() < 4:
        pytest.skip("needs 4 GPUs")
    r = _run(4, {"NEXRT_WAIT_BUDGET_MS": "5000", "NEXRT_CANARY": "1"}, 29613, script="cp_worker.py")
    assert r.returncode == 0 and "CP_WORKER_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


def test_context_parallel_tp2():
    """2 ranks, 1 kv head: one context-parallel group of 2 (the same worker; needs half the GPUs)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    r = _run(2, {"NEXRT_WAIT_BUDGET_MS": "5000", "NEXRT_CANARY": "1"}, 29614, script="cp_worker.py")
    assert r.returncode == 0 and "CP_WORKER_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


def test_allreduce_ops():
    """The packet and block all-reduce protocols as operators: rank-ordered bits, determinism under skew, a silent peer."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    world = 4 if torch.cuda.device_count() >= 4 else 2
    r = _run(world, {"NCCL_NVLS_ENABLE": "0"}, 29615, script="ar_worker.py")
    assert r.returncode == 0 and "AR_WORKER_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


def test_speculative_drafts_tp2():
    """MTP draft layer and DFlash block draft on 2 ranks against their CPU oracles (draft K/V, draft ids)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    r = _run(2, {"NEXRT_WAIT_BUDGET_MS": "5000"}, 29616, script="spec_worker.py")
    assert r.returncode == 0 and "SPEC_WORKER_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


def test_tp8_matches_oracle():
    """All eight ranks: single-row and multi-row logits, the generated stream and the wide prefill against the CPU oracle on a
    shrunk geometry that splits 8 ways (the deployment's world size; the other tests stop at 2 and 4)."""
    if torch.cuda.device_count() < 8:
        pytest.skip("needs 8 GPUs")
    if os.environ.get("NEXRT_RUN_TP8_TEST", "0") != "1":
        pytest.skip("eight-rank run is opt-in (NEXRT_RUN_TP8_TEST=1): it holds a whole node")
    r = _run(8, {"NEXRT_WAIT_BUDGET_MS": "5000", "NEXRT_TEST_GEOMETRY": "tp8"}, 29617)
    assert r.returncode == 0 and "TP_WORKER_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
