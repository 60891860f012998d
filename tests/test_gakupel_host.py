"""Host-side parts of the Gakupel family that need no GPU: configuration reading, the architecture registry, the flat-tensor loader's
strictness, and the oracle's own consistency (layer norm, the sink, the distance bias, the stabilised matrix memory, the grouped
choice of experts, causality of the whole model)."""
import math

import pytest
import torch

from evo_b200.gakupel import Gakupel, GakupelConfig
from evo_b200.models import ARCHITECTURES, load_model_dir, read_architecture
from evo_b200.stream_model import StreamDecoder
from oracle import gakupel_oracle as O
from tests.test_zaverax_host import _write_checkpoint

F64 = torch.float64


def test_config_reads_every_size_and_constant():
    d = O.make_config(layers=("delta", "attention", "parallel", "attention"), mlps=("moe", None, "dense", "moe"), width=104, vocab=77, ff=58, eps=3e-6,
                      att_heads=6, att_kv_heads=3, att_dim=10, rot_dims=6, rot_base=777.0, att_scale=0.31,
                      left_heads=8, left_kv_heads=2, left_dim=20, left_vdim=6, left_scale_qk=0.2, temp_coef=0.7, temp_every=5, left_scale=1.1, right_scale=0.4,
                      mem_heads=3, mem_dim=7, mem_vdim=9, gate_cap=4.5, heads=6, kv_heads=3, dim=10, vdim=14, taps=2,
                      experts=9, top=2, groups=3, keep=1, router_scale=2.5, expert_ff=12, shared_ff=20)
    c = GakupelConfig.from_dict(d)
    assert (c.width, c.vocab_size, c.eps, len(c.runs)) == (104, 77, 3e-6, 4)
    m, a, p = c.layers[0].delta, c.layers[1].attention, c.layers[2]
    assert (m.heads, m.kv_heads, m.dim, m.vdim, m.taps) == (6, 3, 10, 14, 2)
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.scale, a.rot_dims, a.rot_base, a.q_temp_every) == (6, 3, 10, 10, 0.31, 6, 777.0, 0)
    l, r = p.attention, p.memory
    assert (l.heads, l.kv_heads, l.dim, l.vdim, l.scale, l.rot_dims, l.q_temp_coef, l.q_temp_every) == (8, 2, 20, 6, 0.2, 0, 0.7, 5)
    assert (r.heads, r.dim, r.vdim, r.gate_cap, p.left_scale, p.right_scale) == (3, 7, 9, 4.5, 1.1, 0.4)
    f = c.layers[0].mlp
    assert (f.kind, f.ff, f.experts, f.top, f.groups, f.keep, f.router_scale, f.shared_ff) == ("moe", 12, 9, 2, 3, 1, 2.5, 20)
    assert c.layers[1].mlp is None and (c.layers[2].mlp.kind, c.layers[2].mlp.ff) == ("dense", 58)
    shapes = c.tensor_shapes()
    assert shapes == O.tensor_shapes(d)
    assert shapes["l1.mix.q.norm"] == (10,) and shapes["l2.mix.left.q.norm"] == (160,) and shapes["l2.mix.right.norm"] == (27,) and shapes["l3.dwa"] == (5,)
    assert "l1.norm2" not in shapes and "l1.mix.v" not in shapes and c.unused_tensor_names == ("l1.norm2", "l1.norm2.b")
    # what a configuration does not mention does not exist: no rotation, no temperature, no groups, no always-on expert
    bare = O.make_config(layers=("attention", "parallel"), mlps=("moe", "moe"), rot_dims=0, temp_every=0, groups=0, shared_ff=0)
    b = GakupelConfig.from_dict(bare)
    assert b.layers[0].attention.rot_dims == 0 and b.layers[1].attention.q_temp_every == 0 and (b.layers[0].mlp.groups, b.layers[0].mlp.shared_ff) == (0, 0)
    assert "l0.mlp.shared.sg" not in b.tensor_shapes()
    for key, value, err in (("type", "conv", NotImplementedError), ("mlp", {"kind": "sparse"}, NotImplementedError)):
        bad = O.make_config()
        bad["layers"][0][key] = value
        with pytest.raises(err):
            GakupelConfig.from_dict(bad)
    with pytest.raises(ValueError):
        GakupelConfig.from_dict(O.make_config(experts=8, groups=3))
    with pytest.raises(ValueError):
        GakupelConfig.from_dict(O.make_config(experts=8, groups=4, keep=1, top=3))
    with pytest.raises(ValueError):
        GakupelConfig.from_dict(O.make_config(att_heads=5, att_kv_heads=2))


def test_registry_picks_the_class_and_the_loader_is_strict(tmp_path):
    cfg = O.make_config()
    W = O.random_weights(cfg, seed=1)
    _write_checkpoint(tmp_path / "ok", cfg, W)
    arch, read = read_architecture(str(tmp_path / "ok"))
    assert arch == "Gakupel" and read["width"] == cfg["width"] and torch.float32 in ARCHITECTURES[arch][1]
    model = load_model_dir(str(tmp_path / "ok"))
    assert isinstance(model, Gakupel) and isinstance(model, StreamDecoder) and model.ingest_stats["tensors"] == len(W)
    assert all(torch.equal(model.weights[k], W[k]) for k in W)
    missing = dict(W)
    missing.pop("l0.mix.left.r2")
    _write_checkpoint(tmp_path / "missing", cfg, missing)
    with pytest.raises(RuntimeError, match="Missing"):
        load_model_dir(str(tmp_path / "missing"))
    _write_checkpoint(tmp_path / "shape", cfg, dict(W, **{"l2.dwa": W["l2.dwa"][:-1].contiguous()}))
    with pytest.raises(RuntimeError, match="size mismatch"):
        load_model_dir(str(tmp_path / "shape"))
    with pytest.raises(NotImplementedError):
        load_model_dir(str(tmp_path / "ok"), dtype=torch.float16)
    # a layer without feed-forward may still carry its second norm: it is not read
    cfg2 = O.make_config(layers=("delta",), mlps=(None,))
    W2 = O.random_weights(cfg2, seed=2)
    W2["l0.norm2"] = W2["l0.norm2.b"] = W2["l0.norm1"].clone()
    _write_checkpoint(tmp_path / "spare", cfg2, W2)
    assert "l0.norm2" not in load_model_dir(str(tmp_path / "spare")).weights


def test_model_refuses_to_run_without_cuda():
    from evo_b200 import _lib
    cfg = O.make_config()
    m = Gakupel(GakupelConfig.from_dict(cfg))
    m.load_state_dict(O.random_weights(cfg))
    with pytest.raises(RuntimeError):
        m.load_state_dict({"embed": torch.zeros(2, 2)})
    with pytest.raises(_lib.EvoError, match="no CPU"):
        m(torch.zeros(1, 4, dtype=torch.long))
    rnd = Gakupel(GakupelConfig.from_dict(cfg)).init_random(seed=3)
    assert set(rnd.weights) == set(O.tensor_shapes(cfg)) and all(torch.isfinite(v.float()).all() for v in rnd.weights.values())
    assert m.fir_taps == 3


def test_oracle_norm_sink_and_distance_bias():
    u = torch.tensor([[1.0, 2.0, 3.0, 6.0]], dtype=F64)
    y = O.layer_norm(u, torch.full((4,), 2.0, dtype=F64), torch.full((4,), 0.5, dtype=F64), 0.0)
    assert torch.allclose(y.mean(), torch.tensor(0.5, dtype=F64)) and torch.allclose(((y - 0.5) / 2).pow(2).mean(), torch.tensor(1.0, dtype=F64))
    # one token, zero score: the sink takes half of the weight; far keys lose r1 ln(1 + r2 d)
    cfg = O.make_config(layers=("parallel",), mlps=(None,), temp_every=0)
    m = cfg["layers"][0]["mixer"]["left"]
    H, G, dk, dv, D = m["heads"], m["kv_heads"], m["dim"], m["vdim"], cfg["width"]
    w = {"q": torch.zeros(H * dk, D, dtype=F64), "k": torch.randn(G * dk, D, dtype=F64), "v": torch.randn(G * dv, D, dtype=F64),
         "q.norm": torch.ones(H * dk, dtype=F64), "k.norm": torch.ones(G * dk, dtype=F64), "r1": torch.full((H,), 2.0, dtype=F64), "r2": torch.full((H,), 0.5, dtype=F64),
         "o": torch.eye(D, H * dv, dtype=F64)}
    h = torch.randn(3, D, dtype=F64)
    out = O.biased_sink_attention(h, w, m, 1e-6)
    v = (h @ w["v"].T).view(3, G, dv)
    assert torch.allclose(out[0, :dv], 0.5 * v[0, 0])
    e = torch.tensor([math.exp(-2.0 * math.log(1 + 0.5 * d)) for d in (2, 1, 0)], dtype=F64)          # scores are 0: only the bias is left
    assert torch.allclose(out[2, :dv], (e / (1 + e.sum())) @ v[:, 0])


def test_oracle_matrix_memory_is_the_unstabilised_recurrence():
    """The running maximum only rescales: o equals C^T q / max(|n.q|, 1) of the plain sums C = sum_s (prod f) e^i k v^T (while they fit a double)."""
    cfg = O.make_config(layers=("parallel",), mlps=(None,), mem_heads=1, mem_dim=5, mem_vdim=4, gate_cap=3.0)
    m = cfg["layers"][0]["mixer"]["right"]
    D, T = cfg["width"], 12
    g = torch.Generator().manual_seed(0)
    w = {n: torch.randn(s, D, generator=g, dtype=F64) / math.sqrt(D) for n, s in (("q", 5), ("k", 5), ("v", 4), ("g", 4))}
    w.update({"i": torch.randn(1, D, generator=g, dtype=F64), "f": torch.randn(1, D, generator=g, dtype=F64), "i.b": torch.zeros(1, dtype=F64), "f.b": torch.ones(1, dtype=F64),
              "norm": torch.ones(4, dtype=F64), "o": torch.eye(D, 4, dtype=F64)})
    h = torch.randn(T, D, generator=g, dtype=F64)
    got = O.matrix_memory(h, w, m, 1e-6)[:, :4]
    q, k, v = (h @ w["q"].T) * 5 ** -0.5, h @ w["k"].T, h @ w["v"].T
    ig = 3.0 * torch.tanh((h @ w["i"].T)[:, 0] / 3.0)
    fg = torch.nn.functional.logsigmoid(3.0 * torch.tanh(((h @ w["f"].T)[:, 0] + 1.0) / 3.0))
    Cm, n = torch.zeros(5, 4, dtype=F64), torch.zeros(5, dtype=F64)
    for t in range(T):
        Cm = torch.exp(fg[t]) * Cm + torch.exp(ig[t]) * torch.outer(k[t], v[t])
        n = torch.exp(fg[t]) * n + torch.exp(ig[t]) * k[t]
        o = (Cm.T @ q[t]) / (max(abs(float(n @ q[t])), 1.0))
        want = O.rms(o[None], 1e-6)[0] * torch.sigmoid(h[t] @ w["g"].T)
        assert torch.allclose(got[t], want, rtol=1e-4, atol=1e-6), t


def test_oracle_router_keeps_groups_and_normalises():
    D = 6
    w = {"router": torch.zeros(8, D, dtype=F64), "correction": torch.tensor([0.9, 0.0, 0.0, 0.0, 0.5, 0.45, 0.3, 0.35], dtype=F64)}
    h = torch.zeros(1, D, dtype=F64)                        # every score is sigmoid(0) = 1/2; the corrections alone decide
    r = {"experts": 8, "top": 2, "scale": 3.0, "groups": {"count": 4, "keep": 1}}
    # group sums of the two largest selection scores: (1.4+.5, 1.0, .5+.5+.95, .5+.5+.65) -> group 2 wins although expert 0 is the single best
    got = O.route(h, w, r)[0]
    assert got.nonzero().flatten().tolist() == [4, 5] and torch.allclose(got[[4, 5]], torch.tensor([1.5, 1.5], dtype=F64))
    r["groups"]["keep"] = 4
    assert O.route(h, w, r)[0].nonzero().flatten().tolist() == [0, 4]
    del r["groups"]
    assert O.route(h, w, r)[0].nonzero().flatten().tolist() == [0, 4]
    # negative selection scores inside a kept group still beat every expert outside it
    w["correction"] = torch.tensor([-3.0, -4.0, -0.9, -0.8, -0.7, -5.0, -0.6, -0.65], dtype=F64)
    r["groups"] = {"count": 4, "keep": 1}
    assert O.route(h, w, r)[0].nonzero().flatten().tolist() == [6, 7]


def test_oracle_model_is_causal_and_mixes_earlier_layers():
    cfg = O.make_config()
    W = O.random_weights(cfg, seed=4)
    tokens = torch.randint(0, cfg["vocab"], (20,), generator=torch.Generator().manual_seed(1)).tolist()
    full = O.forward(tokens, W, cfg)
    assert torch.allclose(O.forward(tokens[:9], W, cfg), full[:9], atol=1e-9)
    # with the mix of the last layer set to (1, 0, ..., 0) the model's output is the final norm of the embedding rows
    W2 = dict(W)
    n = len(cfg["layers"])
    W2[f"l{n - 1}.dwa"] = torch.tensor([1.0] + [0.0] * n).to(torch.bfloat16)
    w = {k: v.double() for k, v in W2.items()}
    want = O.layer_norm(w["embed"][torch.tensor(tokens)], w["final.norm"], w["final.norm.b"], cfg["norm"]["eps"]) @ w["head"].T
    assert torch.allclose(O.forward(tokens, W2, cfg), want, atol=1e-9)
