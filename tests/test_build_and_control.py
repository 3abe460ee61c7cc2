"""Build helper and control-block ABI (reference tests/test_kernel_build.py, m4_control drift check)."""

import os
import time

import pytest

from nexrt_b200 import build as B
from nexrt_b200.runtime import control as C


def test_sources_and_arch_flags():
    names = {p.name for p in B.sources()}
    assert {"gdn.cu", "attn.cu", "moe.cu", "head.cu", "oproj.cu", "step.cu"} <= names
    assert B.ARCH_FLAGS == ["-gencode", "arch=compute_100a,code=sm_100a"] and "-lineinfo" in B.NVCC_FLAGS


def test_stale_on_header_mtime(tmp_path):
    src, hdr, out = tmp_path / "k.cu", tmp_path / "h.cuh", tmp_path / "k.o"
    hdr.write_text("// h\n")
    src.write_text('#include "h.cuh"\n')
    out.write_text("obj")
    future = time.time() + 100
    os.utime(out, (future, future))
    assert B.is_fresh(out, src)
    os.utime(hdr, (future + 50, future + 50))
    assert not B.is_fresh(out, src)


def test_refuses_symlinked_and_escaping_paths(tmp_path):
    root = tmp_path / "root"
    root.mkdir()
    (tmp_path / "elsewhere").mkdir()
    link = root / "link"
    link.symlink_to(tmp_path / "elsewhere")
    with pytest.raises(RuntimeError):
        B.validate_build_path(link / "x.o", root)
    with pytest.raises(RuntimeError):
        B.validate_build_path(tmp_path / "elsewhere" / "x.o", root)
    assert B.validate_build_path(root / "x.o", root) == root / "x.o"


def test_compiler_failure_leaves_no_partial_file(monkeypatch, tmp_path):
    src = tmp_path / "bad.cu"
    src.write_text("int x;\n")
    monkeypatch.setattr(B, "BUILD_ROOT", tmp_path / "b")
    (tmp_path / "b").mkdir()

    class P:
        returncode, stdout, stderr = 1, "", "boom"

    monkeypatch.setattr(B.subprocess, "run", lambda *a, **k: P())
    with pytest.raises(RuntimeError):
        B.compile_object(src)
    assert list((tmp_path / "b").iterdir()) == []


def test_control_abi_matches_header(tmp_path):
    C.check_abi()
    drift = tmp_path / "common.cuh"
    text = (B.CSRC / "common.cuh").read_text().replace("kCtlPending = 3", "kCtlPending = 7")
    drift.write_text(text)
    with pytest.raises(RuntimeError):
        C.check_abi(drift)


def test_ring_no_alias_law():
    assert C.ring_no_alias(8, 16, 9) and C.ring_no_alias(4, 16, 5) and C.ring_no_alias(1, 16, 2)
    assert not C.ring_no_alias(8, 16, 8) and not C.ring_no_alias(8, 10, 9)
    assert C.state_slot(9, 9) == 0 and C.conv_slot(17, 16) == 1


def test_graph_capture_holds_the_garbage_collector(monkeypatch):
    """The capture helper collects first and keeps the cyclic collector off while the capture runs."""
    import contextlib
    import gc

    import torch

    from nexrt_b200.runtime import capture

    seen = {}

    @contextlib.contextmanager
    def fake_graph(graph, stream=None):
        seen["inside_enter"] = gc.isenabled()
        yield
        seen["inside_exit"] = gc.isenabled()

    monkeypatch.setattr(torch.cuda, "graph", fake_graph)
    assert gc.isenabled()
    with capture.graph_capture(object(), object()):
        seen["body"] = gc.isenabled()
    assert seen == {"inside_enter": False, "body": False, "inside_exit": False} and gc.isenabled()
    with pytest.raises(RuntimeError):
        with capture.graph_capture(object(), object()):
            raise RuntimeError("launch failed")
    assert gc.isenabled()


def test_every_entry_point_has_a_matching_ctypes_prototype():
    """ABI audit: each ``int nexrt_*(...)`` of ``csrc/api.h`` (and of the ``extern "C"`` definitions in the sources) has a
    ctypes prototype with the same number of arguments, and no prototype names an entry point that does not exist."""
    import re
    from pathlib import Path

    from nexrt_b200.ops import lib as L

    csrc = Path(L.__file__).resolve().parent.parent / "csrc"
    text = (csrc / "api.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    declared = {}
    for name, args in re.findall(r"\bint\s+(nexrt_\w+)\s*\(([^;{]*?)\)\s*;", text, flags=re.S):
        args = args.strip()
        declared[name] = 0 if args in ("", "void") else len([a for a in args.split(",") if a.strip()])
    defined = set()
    for src in csrc.glob("*.cu"):
        body = src.read_text()
        defined.update(re.findall(r"\b(?:int|size_t|unsigned long long)\s+(nexrt_\w+)\s*\(", body))
    protos = dict(L._PROTOTYPES)
    assert protos, "no prototypes found"
    missing = [n for n in protos if n not in defined]
    assert not missing, f"prototypes without a definition in csrc: {missing}"
    wrong = {n: (len(protos[n]), declared[n]) for n in protos if n in declared and len(protos[n]) != declared[n]}
    assert not wrong, f"argument count differs between ops/lib.py and csrc/api.h (prototype, header): {wrong}"
    undeclared = [n for n in protos if n not in declared]
    assert not undeclared, f"entry points without a declaration in api.h: {undeclared}"
