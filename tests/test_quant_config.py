"""Host-only checks of the quantiser, geometry, sharding and checkpoint layout."""

import pytest
import torch

from nexrt_b200.config import ShardSpec, full_config, shrunk_config
from nexrt_b200.quant import FP8_MAX, act_quant, dequantize_blockwise, fold_requant, quantize_blockwise
from nexrt_b200.weights import load_checkpoint, normalise_scale_names, random_checkpoint, save_checkpoint, shard_model


def test_block_quant_roundtrip_error():
    g = torch.Generator().manual_seed(0)
    w = torch.randn(256, 384, generator=g) * 0.02
    q, s = quantize_blockwise(w)
    assert q.dtype == torch.float8_e4m3fn and s.shape == (2, 3)
    back = dequantize_blockwise(q, s)
    assert float((back - w).abs().max()) <= float(w.abs().max()) / 16 + 1e-9
    assert float(q.float().abs().max()) <= FP8_MAX


def test_block_quant_ragged_edges():
    w = torch.randn(130, 200)
    q, s = quantize_blockwise(w)
    assert q.shape == w.shape and s.shape == (2, 2)
    assert torch.isfinite(dequantize_blockwise(q, s)).all()


def test_fold_requant_matches_dequant_times_gamma():
    w = torch.randn(128, 256) * 0.02
    q, s = quantize_blockwise(w)
    gamma = 1.0 + 0.1 * torch.randn(256)
    q2, s2 = fold_requant(q, s, gamma)
    want = dequantize_blockwise(q, s) * gamma
    got = dequantize_blockwise(q2, s2)
    assert float((got - want).norm() / want.norm()) < 0.05


def test_act_quant_shapes():
    x = torch.randn(3, 512)
    q, s = act_quant(x)
    assert q.shape == (3, 512) and s.shape == (3, 4)
    with pytest.raises(ValueError):
        act_quant(torch.randn(2, 100))


def test_full_geometry_matches_reference_constants():
    c = full_config()
    assert (c.hidden, c.vocab, c.n_layers) == (4096, 248320, 60)
    assert c.n_full == 15 and c.n_linear == 45
    assert c.layer_types[3] == "full" and c.layer_types[0] == "linear"
    assert c.cache_len == 256 * 1024 + 1024
    s = ShardSpec(c, 8, 5)
    assert (s.q_heads, s.kv_heads, s.kv_head0, s.cp_size, s.cp_rank) == (4, 1, 1, 4, 1)
    assert s.gdn_front_rows == 2560 and s.attn_front_rows == 2560 and s.inter == 128 and s.vocab == 31040
    assert s.cp_group == (4, 5, 6, 7)


@pytest.mark.parametrize("tp", [1, 2, 4, 8])
def test_shard_spec_parametric(tp):
    c = full_config()
    total_q = sum(ShardSpec(c, tp, r).q_heads for r in range(tp))
    assert total_q == c.n_q_heads
    assert ShardSpec(c, tp, 0).inter * tp == c.moe_inter
    assert c.truncated(4).n_layers == 4


def test_shrunk_config_limits():
    c = shrunk_config()
    assert c.supports_tp(2) and not c.supports_tp(4)
    with pytest.raises(ValueError):
        ShardSpec(c, 3, 0)


def test_checkpoint_roundtrip_and_sharding(tmp_path):
    cfg = shrunk_config()
    ck = random_checkpoint(cfg, 0)
    save_checkpoint(ck, cfg, tmp_path)
    back = load_checkpoint(cfg, tmp_path)
    assert set(back) == set(ck)
    for k in ck:
        assert torch.equal(back[k].view(torch.uint8) if back[k].dtype == torch.float8_e4m3fn else back[k],
                           ck[k].view(torch.uint8) if ck[k].dtype == torch.float8_e4m3fn else ck[k])
    # the other checkpoint spelling of the scale tensors is accepted
    alias = {k[: -len("_inv")] if k.endswith("weight_scale_inv") else k: v for k, v in ck.items()}
    m_alias = shard_model(alias, cfg, 2, 1, "cpu")
    m = shard_model(ck, cfg, 2, 1, "cpu")
    assert torch.equal(m["layers"][0]["mixer"]["front_s"], m_alias["layers"][0]["mixer"]["front_s"])
    assert set(normalise_scale_names(alias)) == set(ck)
    # shards tile the global tensors
    s0, s1 = shard_model(ck, cfg, 2, 0, "cpu"), m
    o = ck["model.language_model.layers.1.self_attn.o_proj.weight"].view(torch.uint8)
    got = torch.cat([s0["layers"][1]["mixer"]["out_w"].view(torch.uint8), s1["layers"][1]["mixer"]["out_w"].view(torch.uint8)], 1)
    assert torch.equal(got, o)
    assert s0["layers"][0]["moe"]["w13"].shape == (cfg.n_experts + 1, 2 * 128, cfg.hidden)
    assert s0["head"]["lm_head"].shape == (cfg.vocab // 2, cfg.hidden)


def test_wide_prefill_down_split_gives_every_range_work():
    """The expert down product of the wide prefill path is split along K so that no CTA walks more than 64 blocks and no
    range is empty (the kernel derives its ranges as ceil(blocks / split) per CTA)."""
    from nexrt_b200.prefill_wide import down_split

    assert down_split(513, 32, 148) == 9          # 513 experts x one 128-wide block, TP = 8 shard: 57 blocks per CTA, 288 CTAs
    assert down_split(1, 8, 148) == 1
    for k_blocks in list(range(1, 200)) + [513, 1026, 4104]:
        for tiles in (1, 8, 32, 64):
            ks = down_split(k_blocks, tiles, 148)
            per = -(-k_blocks // ks)
            assert per <= 64 and -(-k_blocks // per) == ks and 1 <= ks <= k_blocks


def test_oracle_with_fp8_activations_quantifies_the_wide_prefill_rounding():
    """The oracle can round the input of every FP8 projection to one e4m3 plane, which is the wide prefill path's arithmetic.
    On the shrunk random-init model that moves the first attention layer's keys by about 11 % (the deviation the GPU test
    of the wide path sees against the exact 8-row path) while the recurrent state of the layer before moves by a few
    per cent: small per projection, compounding through routing and normalisation."""
    from nexrt_b200.models.reference import RefModel, synthetic_prompt
    from nexrt_b200.testing import shrunk_checkpoint

    cfg, ckpt = shrunk_checkpoint(0)
    exact, rounded = RefModel(cfg, ckpt), RefModel(cfg, ckpt, fp8_activations=True)
    prompt = synthetic_prompt(cfg.vocab, 24, seed=5)
    for t in prompt:
        exact.step(t)
        rounded.step(t)
    rel = lambda a, b: float((a - b).norm() / b.norm())
    gdn = rel(rounded.states[0].state, exact.states[0].state)
    keys = rel(torch.stack(rounded.states[1].k, 1), torch.stack(exact.states[1].k, 1))
    assert 0.005 < gdn < 0.1 and 0.02 < keys < 0.3, (gdn, keys)


def test_wide_prefill_covers_every_tensor_parallel_degree_of_the_full_model():
    from types import SimpleNamespace

    from nexrt_b200.config import ShardSpec, full_config, shrunk_config
    from nexrt_b200.prefill_wide import supported

    for cfg, degrees in ((full_config(), (1, 2, 4, 8)), (shrunk_config(), (1, 2))):
        for tp in degrees:
            eng = SimpleNamespace(cfg=cfg, spec=ShardSpec(cfg, tp, 0), max_rows=8)
            assert supported(eng), (cfg.name, tp)
    # the sequential parts run eight rows at a time on the step kernels' rings: an engine built for fewer rows is out
    assert not supported(SimpleNamespace(cfg=full_config(), spec=ShardSpec(full_config(), 8, 0), max_rows=4))


def test_activation_split_terms_add_up():
    """CPU statement of the wide prefill's quantisers: one, two and three e4m3 terms reproduce the value to 2^-4, 2^-8 and
    2^-12 per element, each term's scale is the first one's divided by 16^p, and one term is the plain quantiser."""
    from nexrt_b200.quant import act_quant_terms

    g = torch.Generator().manual_seed(5)
    x = torch.randn(6, 384, generator=g) * torch.logspace(-3, 2, 6)[:, None]
    x[2, 128:256] = 0.0                                   # an all-zero block keeps a finite scale and zero terms
    deq = lambda q, s, terms: sum(
        (q[p * 6 : (p + 1) * 6].float().reshape(6, -1, 128) * s[p * 6 : (p + 1) * 6, :, None]).reshape(6, -1) for p in range(terms))
    q1, s1 = act_quant_terms(x, 1)
    q0, s0 = act_quant(x)
    assert torch.equal(s1[x.abs().reshape(6, 3, 128).amax(-1) > 0], s0[x.abs().reshape(6, 3, 128).amax(-1) > 0])
    for terms, bound in ((1, 2.0 ** -4), (2, 2.0 ** -8), (3, 2.0 ** -12)):
        q, s = act_quant_terms(x, terms)
        assert q.shape == (terms * 6, 384) and s.shape == (terms * 6, 3)
        err = (deq(q, s, terms) - x).abs()
        # relative to each value, except below e4m3's subnormal step of the LAST term's scale
        floor = (s[(terms - 1) * 6 :, :, None] * 2.0 ** -10).expand(6, 3, 128).reshape(6, -1)
        assert bool((err <= bound * x.abs() + floor).all()), (terms, float((err / x.abs().clamp_min(1e-30)).max()))
        for p in range(1, terms):
            assert torch.equal(s[p * 6 : (p + 1) * 6] * 16.0 ** p, s[:6])
    assert bool((deq(*act_quant_terms(x, 3), 3)[2, 128:256] == 0).all())


def _flat(x, prefix=""):
    if isinstance(x, dict):
        for k, v in x.items():
            yield from _flat(v, f"{prefix}.{k}")
    elif isinstance(x, (list, tuple)):
        for i, v in enumerate(x):
            yield from _flat(v, f"{prefix}.{i}")
    elif isinstance(x, torch.Tensor):
        yield prefix, x


def _same(a, b):
    fa, fb = dict(_flat(a)), dict(_flat(b))
    assert fa.keys() == fb.keys()
    for k in fa:
        x, y = fa[k], fb[k]
        assert x.dtype == y.dtype and x.shape == y.shape, k
        assert torch.equal(x.view(torch.uint8) if x.element_size() == 1 else x, y.view(torch.uint8) if y.element_size() == 1 else y), k


def test_streaming_loader_equals_the_eager_one_and_reads_each_tensor_once(tmp_path):
    """``LayerFiles`` is the layer directory as a lazy mapping: sharding from it gives the eager loader's tensors bit for
    bit (both scale names), no tensor is read twice, shapes come from the header, unknown names raise ``KeyError``."""
    from nexrt_b200.weights import LayerFiles, load_rank_model

    cfg = shrunk_config()
    ck = random_checkpoint(cfg, 3)
    ck = {(k[: -len("_inv")] if k.endswith("weight_scale_inv") and ".layers.1." in k else k): v for k, v in ck.items()}   # one layer under the other name
    save_checkpoint(ck, cfg, tmp_path)
    eager = shard_model(load_checkpoint(cfg, tmp_path), cfg, 2, 1, "cpu", cp=True)
    _same(load_rank_model(cfg, tmp_path, 2, 1, "cpu", cp=True), eager)
    files = LayerFiles(cfg, tmp_path, prefault=False)
    assert len(files) == len(ck) and set(files) == set(ck)
    key = "model.language_model.embed_tokens.weight"
    assert files.shape(key) == tuple(ck[key].shape) and files.reads == 0
    shard_model(files, cfg, 2, 0, "cpu")
    assert 0 < files.reads <= len(ck)                    # every tensor at most once per rank
    with pytest.raises(KeyError):
        files["model.language_model.layers.99.input_layernorm.weight"]
    files.close()


def test_prefault_reads_the_file_and_leaves_it_alone(tmp_path):
    """Warming the page cache is read-only (reference tests/test_weight_loading.py: test_prefault_preserves_checkpoint)."""
    from nexrt_b200.weights import prefault_file

    path = tmp_path / "weights.safetensors"
    contents = b"original checkpoint" * ((20 << 20) // 19 + 1)
    path.write_bytes(contents)
    before = path.stat()
    assert prefault_file(path) == len(contents)
    assert path.read_bytes() == contents and path.stat().st_mtime_ns == before.st_mtime_ns and path.stat().st_size == before.st_size
    assert list(tmp_path.iterdir()) == [path]


def test_draft_loaders_read_files_and_check_geometry(tmp_path):
    """MTP weights come from ``mtp.safetensors`` of the layer directory and share the target's resident head; the DFlash
    draft comes from its own ``model.safetensors`` after a shape check of every tensor against the fixed geometry
    (reference tests/test_mtp_weight_sharing.py, dflash/weights.py:117-142)."""
    from safetensors.torch import save_file

    from nexrt_b200.dflash.config import shrunk_dflash_config
    from nexrt_b200.dflash.weights import check_dflash_checkpoint, load_dflash_files, load_dflash_shard, random_dflash_checkpoint
    from nexrt_b200.mtp.weights import load_mtp_files, random_mtp_checkpoint, shard_mtp

    cfg = shrunk_config()
    ck = random_checkpoint(cfg, 1)
    mtp = random_mtp_checkpoint(cfg, 7)
    save_checkpoint({**ck, **mtp}, cfg, tmp_path)
    head = shard_model(ck, cfg, 2, 1, "cpu")["head"]
    got = load_mtp_files(cfg, tmp_path, 2, 1, "cpu", head)
    _same(got, shard_mtp(mtp, cfg, 2, 1, "cpu", head))
    assert got["head"]["lm_head"] is head["lm_head"] and got["head"]["embed"] is head["embed"]      # shared, not copied
    with pytest.raises(ValueError, match="not resident"):
        shard_mtp(mtp, cfg, 2, 1, "cpu", {"final_ln": head["final_ln"], "lm_head": None, "embed": head["embed"]})
    (tmp_path / "mtp.safetensors").unlink()
    with pytest.raises(FileNotFoundError):
        load_mtp_files(cfg, tmp_path, 2, 1, "cpu", head)

    dc = shrunk_dflash_config(cfg)
    dck = random_dflash_checkpoint(dc, 11)
    path = tmp_path / "model.safetensors"
    save_file({k: v.contiguous() for k, v in dck.items()}, str(path))
    _same(load_dflash_files(dc, 2, 0, "cpu", path), load_dflash_shard(dck, dc, 2, 0, "cpu"))
    check_dflash_checkpoint(dck, dc)
    bad = dict(dck)
    bad["layers.0.mlp.up_proj.weight"] = bad["layers.0.mlp.up_proj.weight"][:-1]
    del bad["norm.weight"]
    with pytest.raises(ValueError, match=r"norm.weight: missing.*layers.0.mlp.up_proj.weight: shape"):
        check_dflash_checkpoint(bad, dc)
    save_file({k: v.contiguous() for k, v in bad.items()}, str(path))
    with pytest.raises(ValueError, match="draft geometry"):
        load_dflash_files(dc, 2, 0, "cpu", path)


def _deq(wq, ws):
    """Dequantise a block-scaled FP8 matrix [R, K] with scales [ceil(R/128), K/128] in float64."""
    R, K = wq.shape
    s = ws.double().repeat_interleave(128, 0)[:R].repeat_interleave(128, 1)[:, :K]
    return wq.view(torch.float8_e4m3fn).double() * s


@pytest.mark.parametrize("tp", [1, 2, 4, 8])
def test_rank_shards_compute_what_the_checkpoint_computes(tp):
    """Sharding as a function, for every tensor-parallel degree including the 8-way deployment split: the rank-local
    tensors (rows AND their block scales), put through the layer's algebra and summed / concatenated over the ranks, give
    the full checkpoint's result.  Checks the pairing the kernels rely on - a rank's v / z rows with its out-projection
    columns, its q heads with the kv head GQA assigns them, an expert's gate / up rows with its down columns, the vocab
    rows - which a random-weight benchmark cannot see."""
    from nexrt_b200.config import ShardSpec, shrunk_tp8_config
    from nexrt_b200.weights import PFX

    cfg = shrunk_tp8_config() if tp == 8 else shrunk_config()
    if tp == 4:
        from nexrt_b200.config import shrunk_cp_config

        cfg = shrunk_cp_config()
    ck = random_checkpoint(cfg, 5)
    shards = [shard_model(ck, cfg, tp, r, "cpu") for r in range(tp)]
    g = torch.Generator().manual_seed(1)
    x = torch.randn(cfg.hidden, generator=g, dtype=torch.float64)
    W = lambda key: _deq(ck[key], ck[key + "_scale_inv"])
    rel = lambda a, b: float((a - b).norm() / b.norm().clamp_min(1e-30))
    lin = next(l for l in range(cfg.n_layers) if cfg.layer_types[l] == "linear")
    att = next(l for l in range(cfg.n_layers) if cfg.layer_types[l] != "linear")

    # gated delta net: sum_r out_r @ (v_r * z_r) == out @ (v * z), with v, z the projections of x
    a = f"{PFX}layers.{lin}.linear_attn."
    kd, vd = cfg.gdn_key_dim, cfg.gdn_value_dim
    qkv, z = W(a + "in_proj_qkv.weight") @ x, W(a + "in_proj_z.weight") @ x
    want = W(a + "out_proj.weight") @ (qkv[2 * kd :] * z)
    got = torch.zeros_like(want)
    for r, sh in enumerate(shards):
        m = sh["layers"][lin]["mixer"]
        pre = _deq(m["front_w"].view(torch.uint8), m["front_s"]) @ x
        kr, vr = kd // tp, vd // tp
        assert rel(pre[:kr], qkv[r * kr : (r + 1) * kr]) < 1e-9 and rel(pre[kr : 2 * kr], qkv[kd + r * kr : kd + (r + 1) * kr]) < 1e-9
        got += _deq(m["out_w"].view(torch.uint8), m["out_s"]) @ (pre[2 * kr : 2 * kr + vr] * pre[2 * kr + vr :])
        nv = cfg.gdn_v_heads // tp
        assert torch.equal(m["a_log"], ck[a + "A_log"].float()[r * nv : (r + 1) * nv])
        assert torch.equal(m["ba_w"][:nv].float(), ck[a + "in_proj_b.weight"][r * nv : (r + 1) * nv].to(torch.bfloat16).float())
    assert rel(got, want) < 1e-9

    # attention: every q head of a rank is paired with the kv head GQA gives it, and sum_r o_r @ (q_r * gate_r) == o @ (q * gate)
    a = f"{PFX}layers.{att}.self_attn."
    hd, nq, nkv = cfg.head_dim, cfg.n_q_heads, cfg.n_kv_heads
    qg, k, v = W(a + "q_proj.weight") @ x, W(a + "k_proj.weight") @ x, W(a + "v_proj.weight") @ x
    qg_h = qg.reshape(nq, 2, hd)
    want = W(a + "o_proj.weight") @ (qg_h[:, 0] * qg_h[:, 1]).reshape(-1)
    got = torch.zeros_like(want)
    for r, sh in enumerate(shards):
        spec = ShardSpec(cfg, tp, r)
        m = sh["layers"][att]["mixer"]
        pre = _deq(m["front_w"].view(torch.uint8), m["front_s"]) @ x
        ql, kl = spec.q_heads, spec.kv_heads
        q_r = pre[: ql * 2 * hd].reshape(ql, 2, hd)
        assert rel(q_r, qg_h[r * ql : (r + 1) * ql]) < 1e-9
        for j in range(ql):                                   # GQA: global q head h reads kv head h // (nq / nkv)
            kv_global = (r * ql + j) // (nq // nkv)
            assert spec.kv_head0 <= kv_global < spec.kv_head0 + kl
        k_r = pre[ql * 2 * hd : ql * 2 * hd + kl * hd]
        v_r = pre[ql * 2 * hd + kl * hd :]
        assert rel(k_r, k[spec.kv_head0 * hd : (spec.kv_head0 + kl) * hd]) < 1e-9 and rel(v_r, v[spec.kv_head0 * hd : (spec.kv_head0 + kl) * hd]) < 1e-9
        got += _deq(m["out_w"].view(torch.uint8), m["out_s"]) @ (q_r[:, 0] * q_r[:, 1]).reshape(-1)
        if spec.cp_size > 1:
            # context-parallel front: the query halves of every head that shares this rank's kv head (global head order),
            # then the rank's own gate halves, then k and v
            mc = shard_model(ck, cfg, tp, r, "cpu", cp=True)["layers"][att]["mixer_cp"]
            pc = _deq(mc["front_w"].view(torch.uint8), mc["front_s"]) @ x
            n_all = ql * spec.cp_size
            g0 = spec.cp_group[0] * ql
            assert list(spec.cp_group) == [rr for rr in range(tp) if ShardSpec(cfg, tp, rr).kv_head0 == spec.kv_head0]
            assert rel(pc[: n_all * hd].reshape(n_all, hd), qg_h[g0 : g0 + n_all, 0]) < 1e-9
            assert rel(pc[n_all * hd : (n_all + ql) * hd].reshape(ql, hd), qg_h[r * ql : (r + 1) * ql, 1]) < 1e-9
            assert rel(pc[(n_all + ql) * hd :], torch.cat([k_r, v_r])) < 1e-9
    assert rel(got, want) < 1e-9

    # experts (a routed one and the shared one): sum_r down_r @ (silu(gate_r x) * up_r x) == the expert
    mbase = f"{PFX}layers.{lin}.mlp."
    for e, ep in ((3, mbase + "experts.3."), (cfg.n_experts, mbase + "shared_expert.")):
        want = W(ep + "down_proj.weight") @ (torch.nn.functional.silu(W(ep + "gate_proj.weight") @ x) * (W(ep + "up_proj.weight") @ x))
        got = torch.zeros_like(want)
        for sh in shards:
            m = sh["layers"][lin]["moe"]
            gu = _deq(m["w13"][e].view(torch.uint8), m["w13_s"][e]) @ x
            Il = gu.numel() // 2
            got += _deq(m["w2"][e].view(torch.uint8), m["w2_s"][e]) @ (torch.nn.functional.silu(gu[:Il]) * gu[Il:])
        assert rel(got, want) < 1e-9
    router = torch.cat([ck[mbase + "gate.weight"], ck[mbase + "shared_expert_gate.weight"].reshape(1, -1)], 0).to(torch.bfloat16)
    assert all(torch.equal(sh["layers"][lin]["moe"]["router_w"], router) for sh in shards)

    # vocabulary rows
    assert torch.equal(torch.cat([sh["head"]["lm_head"] for sh in shards], 0), ck["lm_head.weight"].to(torch.bfloat16))


@pytest.mark.parametrize("tp", [1, 2, 4, 8])
def test_draft_shards_compute_what_the_draft_checkpoints_compute(tp):
    """The same functional check for the two draft models: DFlash (bf16 rows / columns, the fc window over the
    concatenated target features, the kv head a rank's q heads attend to) and MTP (the re-quantised fc window)."""
    from nexrt_b200.config import shrunk_tp8_config
    from nexrt_b200.dflash.config import shrunk_dflash_config
    from nexrt_b200.dflash.weights import load_dflash_shard, random_dflash_checkpoint
    from nexrt_b200.mtp.weights import random_mtp_checkpoint, shard_mtp

    from nexrt_b200.config import shrunk_cp_config

    cfg = shrunk_tp8_config() if tp == 8 else (shrunk_cp_config() if tp == 4 else shrunk_config())
    dc = shrunk_dflash_config(cfg)
    dc.validate_kernel_contract(cfg, tp)
    ck = random_dflash_checkpoint(dc, 11)
    shards = [load_dflash_shard(ck, dc, tp, r, "cpu") for r in range(tp)]
    g = torch.Generator().manual_seed(2)
    H, hd = dc.hidden, dc.head_dim
    x = torch.randn(H, generator=g, dtype=torch.float64)
    taps = torch.randn(dc.n_taps * H, generator=g, dtype=torch.float64)
    rel = lambda a, b: float((a - b).norm() / b.norm().clamp_min(1e-30))
    f = lambda k: ck[k].double()
    assert rel(sum(sh["fc"].double() @ taps[sh["win0"] : sh["win0"] + sh["win"]] for sh in shards), f("fc.weight") @ taps) < 1e-12
    p = "layers.0."
    q, k, v = f(p + "self_attn.q_proj.weight") @ x, f(p + "self_attn.k_proj.weight") @ x, f(p + "self_attn.v_proj.weight") @ x
    want_o = f(p + "self_attn.o_proj.weight") @ q
    want_m = f(p + "mlp.down_proj.weight") @ (torch.nn.functional.silu(f(p + "mlp.gate_proj.weight") @ x) * (f(p + "mlp.up_proj.weight") @ x))
    got_o, got_m = torch.zeros_like(want_o), torch.zeros_like(want_m)
    group = dc.n_q_heads // dc.n_kv_heads
    for r, sh in enumerate(shards):
        lw = sh["layers"][0]
        ql, kl = sh["q_local"], sh["kv_local"]
        pre = lw["wqkv"].double() @ x
        q_r, k_r, v_r = pre[: ql * hd], pre[ql * hd : (ql + kl) * hd], pre[(ql + kl) * hd :]
        assert rel(q_r, q[r * ql * hd : (r + 1) * ql * hd]) < 1e-12
        kv0 = (r * ql) // group                               # the kv head of the rank's first q head
        assert all((r * ql + j) // group in range(kv0, kv0 + kl) for j in range(ql))
        assert rel(k_r, k[kv0 * hd : (kv0 + kl) * hd]) < 1e-12 and rel(v_r, v[kv0 * hd : (kv0 + kl) * hd]) < 1e-12
        assert torch.equal(lw["wkv"], lw["wqkv"][ql * hd :])
        got_o += lw["wo"].double() @ q_r
        gu = lw["wgu"].double() @ x
        Il = sh["I_local"]
        got_m += lw["wdown"].double() @ (torch.nn.functional.silu(gu[:Il]) * gu[Il:])
    assert rel(got_o, want_o) < 1e-12 and rel(got_m, want_m) < 1e-12

    # MTP: the fc over [embedding | hidden] is re-quantised once and split by input window
    tck = random_checkpoint(cfg, 1)
    mck = random_mtp_checkpoint(cfg, 7)
    cat = torch.randn(2 * cfg.hidden, generator=g, dtype=torch.float64)
    got = torch.zeros(cfg.hidden, dtype=torch.float64)
    for r in range(tp):
        head = shard_model(tck, cfg, tp, r, "cpu")["head"] if r == 0 else head
        sh = shard_mtp(mck, cfg, tp, r, "cpu", head)
        got += _deq(sh["fc_w"].view(torch.uint8), sh["fc_s"]) @ cat[sh["win0"] : sh["win0"] + sh["win"]]
    fq, fs = quantize_blockwise(mck["mtp.fc.weight"].float())
    assert rel(got, _deq(fq.view(torch.uint8), fs) @ cat) < 1e-9


@pytest.mark.parametrize("tp,cp", [(1, False), (2, False), (8, True)])
def test_direct_rank_initialisation_has_the_layout_of_a_sharded_checkpoint(tp, cp):
    """``random_rank_model`` (what the benchmarks build at full geometry, where no global tensor may exist) must hand the
    engine exactly the structure ``shard_model`` makes from a checkpoint: same keys, shapes and dtypes on every level."""
    from nexrt_b200.config import shrunk_tp8_config
    from nexrt_b200.weights import random_rank_model

    cfg = shrunk_tp8_config() if tp == 8 else shrunk_config()
    a = dict(_flat(random_rank_model(cfg, tp, tp - 1, "cpu", cp=cp)))
    b = dict(_flat(shard_model(random_checkpoint(cfg, 0), cfg, tp, tp - 1, "cpu", cp=cp)))
    assert set(a) == set(b), sorted(set(a) ^ set(b))
    for k in b:
        assert a[k].shape == b[k].shape and a[k].dtype == b[k].dtype, (k, a[k].shape, b[k].shape, a[k].dtype, b[k].dtype)
