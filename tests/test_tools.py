"""Host-side tools: checkpoint splitter, exact-length prompts, corpus builder, chat client parsing,
state-file naming, preflight."""

import json

import pytest
import torch

from nexrt_b200.extract_layers import canonical_key, extract, plan_outputs
from nexrt_b200.extract_state import make_prompt, state_dir
from nexrt_b200.prep_english_docs import clean_turn, collect
from nexrt_b200.real_prompts import build_real_prompt, fixed_suffix_len
from nexrt_b200.serve.bridge_serve import ByteTokenizer
from nexrt_b200.serve.launch import preflight
from nexrt_b200.serve.stream_chat import completion_url, parse_sse, payload
from nexrt_b200.weights import PFX


def _no_mtp(tmp_path):
    """A sharded checkpoint directory without any mtp.* tensor."""
    from safetensors.torch import save_file

    d = tmp_path / "no-mtp"
    d.mkdir()
    save_file({"x.weight": torch.zeros(1)}, str(d / "s.safetensors"))
    (d / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"x.weight": "s.safetensors"}}))
    return d


def test_extract_layers_splits_and_normalises_scale_names(tmp_path):
    from safetensors.torch import load_file, save_file

    src, dst = tmp_path / "src", tmp_path / "dst"
    src.mkdir()
    a = {f"{PFX}layers.0.mlp.gate.weight": torch.ones(2, 2), f"{PFX}layers.0.self_attn.q_proj.weight_scale": torch.ones(1, 1, dtype=torch.bfloat16),
         f"{PFX}embed_tokens.weight": torch.zeros(4, 2)}
    b = {f"{PFX}layers.1.mlp.gate.weight": torch.full((2, 2), 2.0), f"{PFX}layers.1.self_attn.q_proj.weight_scale_inv": torch.ones(1, 1),
         f"{PFX}norm.weight": torch.zeros(2), "lm_head.weight": torch.zeros(4, 2), "mtp.fc.weight": torch.zeros(2, 4)}
    save_file(a, str(src / "model-00001.safetensors"))
    save_file(b, str(src / "model-00002.safetensors"))
    wm = {**{k: "model-00001.safetensors" for k in a}, **{k: "model-00002.safetensors" for k in b}}
    (src / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wm}))
    written = extract(str(src), str(dst), layers=[0, 1], log=lambda *_: None)
    assert set(written) == {"layer.0.safetensors", "layer.1.safetensors", "embed_tokens.safetensors", "norm.safetensors", "lm_head.safetensors", "mtp.safetensors"}
    l0 = load_file(str(dst / "layer.0.safetensors"))
    key = f"{PFX}layers.0.self_attn.q_proj.weight_scale_inv"
    assert key in l0 and l0[key].dtype == torch.float32 and canonical_key("x.weight_scale") == "x.weight_scale_inv"
    assert not list(dst.glob("*.tmp"))
    # the MTP head from a checkpoint of its own: only its mtp.* tensors are taken, under canonical names
    msrc = tmp_path / "mtp-src"
    msrc.mkdir()
    m = {"mtp.fc.weight": torch.full((2, 4), 5.0), "mtp.fc.weight_scale": torch.ones(1, 1, dtype=torch.bfloat16), "ignored.weight": torch.zeros(1)}
    save_file(m, str(msrc / "mtp-00001.safetensors"))
    (msrc / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {k: "mtp-00001.safetensors" for k in m}}))
    written = extract(str(src), str(dst), layers=[0], with_globals=False, log=lambda *_: None, mtp_src=str(msrc))
    assert set(written) == {"layer.0.safetensors", "mtp.safetensors"} and written["mtp.safetensors"] == 2
    got = load_file(str(dst / "mtp.safetensors"))
    assert set(got) == {"mtp.fc.weight", "mtp.fc.weight_scale_inv"} and float(got["mtp.fc.weight"][0, 0]) == 5.0 and got["mtp.fc.weight_scale_inv"].dtype == torch.float32
    assert set(extract(None, str(dst), log=lambda *_: None, mtp_src=str(msrc))) == {"mtp.safetensors"}
    with pytest.raises(KeyError):
        extract(None, str(dst), log=lambda *_: None, mtp_src=str(_no_mtp(tmp_path)))
    with pytest.raises(KeyError):
        plan_outputs(wm, [5])
    with pytest.raises(KeyError):
        plan_outputs({k: v for k, v in wm.items() if k != "lm_head.weight"}, [0])


@pytest.mark.parametrize("L", [16, 64, 257, 3000])
def test_real_prompt_has_exact_length_and_intact_tail(L):
    tok = ByteTokenizer()
    ids = build_real_prompt(L, tok)
    tail = fixed_suffix_len(tok)
    full = tok.apply_chat_template([{"role": "user", "content": "zz"}], tokenize=True, add_generation_prompt=True)
    assert len(ids) == L and ids == build_real_prompt(L, tok) and ids[-tail:] == full[-tail:]
    with pytest.raises(ValueError):
        build_real_prompt(4, tok)


def test_corpus_builder_filters_turns():
    long_text = "word " * 200
    assert clean_turn("short") is None and clean_turn(long_text + "```code```") == long_text.strip()
    assert clean_turn("é" * 1000) is None
    recs = [{"conversations": [{"from": "human", "value": long_text}, {"from": "gpt", "value": long_text}]}, "junk", {"conversations": [{"from": "gpt", "value": long_text}]}]
    assert len(list(collect(recs, 10))) == 1 and len(list(collect(recs, 10 ** 9))) == 2


def test_chat_client_helpers():
    assert completion_url("http://h:1/v1/") == "http://h:1/v1/chat/completions" == completion_url("http://h:1/v1/chat/completions")
    body = payload("m", [{"role": "user", "content": "x"}], "k", 5, seed=3)
    assert body["stream"] and body["cache_key"] == "k" and body["seed"] == 3 and "seed" not in payload("m", [], "k", 5)
    lines = [b": comment\n", b'data: {"a": 1}\n', b"\n", b"data: [DONE]\n", b'data: {"never": 1}\n']
    assert list(parse_sse(iter(lines))) == [{"a": 1}]


def test_state_dir_prompt_and_preflight(tmp_path):
    assert state_dir("/x", 60, 1024).name == "prefill_state_60_1024"
    p = make_prompt(33, 1000)
    assert len(p) == 33 and p == make_prompt(33, 1000) and max(p) < 1000
    rows = {r["check"]: r for r in preflight(3, layers_dir=str(tmp_path), probe_gpu=False)}
    assert not rows["tp degree"]["ok"] and not rows["layer directory"]["ok"] and "embed_tokens" in rows["layer directory"]["detail"]
    assert {r["check"]: r["ok"] for r in preflight(8, probe_gpu=False)}["tp degree"]
    # every layer file is looked for, and a speculative mode reports (without failing) that its draft would be random
    for name in ("embed_tokens", "norm", "lm_head", "layer.0", "layer.1"):
        (tmp_path / f"{name}.safetensors").write_bytes(b"")
    rows = {r["check"]: r for r in preflight(2, layers_dir=str(tmp_path), probe_gpu=False, mode="mtp", n_layers=3)}
    assert not rows["layer directory"]["ok"] and "layer.2" in rows["layer directory"]["detail"] and "1 of 6" in rows["layer directory"]["detail"]
    (tmp_path / "layer.2.safetensors").write_bytes(b"")
    rows = {r["check"]: r for r in preflight(2, layers_dir=str(tmp_path), probe_gpu=False, mode="mtp", n_layers=3)}
    assert rows["layer directory"]["ok"] and rows["MTP draft weights"]["ok"] and "RANDOM" in rows["MTP draft weights"]["detail"]
    (tmp_path / "mtp.safetensors").write_bytes(b"")
    rows = {r["check"]: r for r in preflight(2, layers_dir=str(tmp_path), probe_gpu=False, mode="mtp", n_layers=3)}
    assert "RANDOM" not in rows["MTP draft weights"]["detail"]
    assert "RANDOM" in {r["check"]: r for r in preflight(2, probe_gpu=False, mode="dflash")}["DFlash draft weights"]["detail"]


def test_timeline_collector_groups_launches_of_mixed_grids():
    """Records of one kind may come from launches of different grid sizes (the helper kernels share a list): the
    collector must rebuild each launch from the records of its own grid size, in entry order."""
    import torch

    from nexrt_b200.utils.trace_step import collect

    kinds, slots, words = 3, 16, 9
    buf = torch.zeros(kinds + kinds * slots * words, dtype=torch.int64)
    recs = buf[kinds:].view(kinds, slots, words)

    def rec(kind, slot, cta, grid, t0, t1, t3):
        recs[kind, slot, 0] = cta | (grid << 32)
        recs[kind, slot, 1], recs[kind, slot, 2], recs[kind, slot, 4] = t0, t1, t3

    # kind 1: a 2-CTA launch, then a 3-CTA launch whose first CTA entered before the first launch's second CTA
    rec(1, 0, 0, 2, 100, 110, 150)
    rec(1, 1, 0, 3, 105, 160, 200)
    rec(1, 2, 1, 2, 108, 112, 155)
    rec(1, 3, 1, 3, 120, 161, 210)
    rec(1, 4, 2, 3, 121, 162, 205)
    buf[1] = 5
    # kind 2: one complete single-CTA launch and one record of an unfinished 4-CTA launch (dropped)
    rec(2, 0, 0, 1, 300, 301, 320)
    rec(2, 1, 0, 4, 330, 331, 340)
    buf[2] = 2
    launches = collect(buf, kinds, slots, words)
    assert [(l["kind"], l["grid"], l["exit"]) for l in launches] == [(1, 2, 155), (1, 3, 210), (2, 1, 320)]
    assert launches[1]["wait_first"] == 160 and launches[0]["entry"] == 100


def test_engine_cli_maps_the_reference_modes_to_tools():
    from nexrt_b200.decode_engine import cli_dispatch

    assert cli_dispatch(["--graph", "--layers", "8"]) == ("profile_step", ["--graph", "--layers", "8"])
    assert cli_dispatch(["--profile"]) == ("profile_step", ["--graph", "--leave-one-out"])
    assert cli_dispatch(["--scale", "--nodes", "64"]) == ("launch_floor", ["--nodes", "64"])
    module, args = cli_dispatch(["--cp-sweep", "--rounds", "50"])
    assert module == "bench_modes" and args[0] == "--cases" and "bs1cp:262144" in args[1] and args[-2:] == ["--rounds", "50"]
    assert cli_dispatch(["--cp", "--cases", "bs1cp:8192"]) == ("bench_modes", ["--cases", "bs1cp:8192"])
    assert cli_dispatch(["--steps", "3"]) == ("profile_step", ["--steps", "3"])
