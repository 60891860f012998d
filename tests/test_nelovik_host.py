"""Host-side parts of the Nelovik family that need no GPU: configuration reading, the architecture registry, the flat-tensor loader's
strictness, and the oracle's own consistency (visibility rule, rotation, activation, one-pass form of the delta rule)."""
import math

import pytest
import torch

from evo_b200.models import ARCHITECTURES, load_model_dir, read_architecture
from evo_b200.nelovik import Nelovik, NelovikConfig
from evo_b200.stream_model import StreamDecoder
from oracle import nelovik_oracle as O
from tests.test_zaverax_host import _write_checkpoint


def test_config_reads_every_size_and_constant():
    d = O.make_config(width=104, vocab=77, layers=("delta_7", "parallel", "delta"), ff=58, no_ff_layers=(2,), eps=3e-6, heads=6, kv_heads=3, dim=10, vdim=14, taps=2,
                      att_heads=8, att_kv_heads=2, att_dim=20, att_vdim=6, window=13, pool=5, rot_dims=10, rot_base=777.0, scale=0.31, softcap=9.0,
                      ssd_heads=6, ssd_vdim=4, state=11, groups=3, norm_groups=4, ssd_taps=5)
    c = NelovikConfig.from_dict(d)
    assert (c.width, c.vocab_size, c.eps, len(c.runs)) == (104, 77, 3e-6, 3)
    m, a, s = c.layers[0].delta, c.layers[1].left, c.layers[1].right
    assert c.layers[0].kind == "delta" and (m.heads, m.kv_heads, m.dim, m.vdim, m.taps) == (6, 3, 10, 14, 2)
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.scale, a.softcap, a.window, a.pool, a.rot_dims, a.rot_base) == (8, 2, 20, 6, 0.31, 9.0, 13, 5, 10, 777.0)
    assert (s.heads, s.vdim, s.state, s.groups, s.norm_groups, s.taps, s.inner, s.conv_channels) == (6, 4, 11, 3, 4, 5, 24, 24 + 66)
    assert c.layers[0].ff == 58 and c.layers[2].ff is None
    shapes = c.tensor_shapes()
    assert shapes == O.tensor_shapes(d)
    assert shapes["l1.mix.right.in"] == (2 * 24 + 2 * 33 + 6, 104) and shapes["l1.mix.left.q.norm"] == (160,) and shapes["l0.mix.q.conv"] == (30, 2)
    assert "l2.norm2" not in shapes and "l2.mlp.up" not in shapes and shapes["l0.mlp.act"] == (2,)
    # what a configuration does not mention does not exist: no rotation, no cap, no pooled blocks
    bare = O.make_config(layers=("parallel",))
    left = bare["layers"][0]["mixer"]["left"]
    del left["rot"], left["softcap"], left["mask"]["pool"]
    b = NelovikConfig.from_dict(bare).layers[0].left
    assert (b.rot_dims, b.softcap, b.pool) == (0, 0.0, 0)
    for breakage in ("type", "kind"):
        bad = O.make_config()
        if breakage == "type":
            bad["layers"][0]["type"] = "delta_x"
        else:
            bad["layers"][0]["mlp"]["kind"] = "sparse"
        with pytest.raises(NotImplementedError):
            NelovikConfig.from_dict(bad)


def test_registry_picks_the_class_and_the_loader_is_strict(tmp_path):
    cfg = O.make_config()
    W = O.random_weights(cfg, seed=1)
    _write_checkpoint(tmp_path / "ok", cfg, W)
    arch, read = read_architecture(str(tmp_path / "ok"))
    assert arch == "Nelovik" and read["width"] == cfg["width"] and torch.float32 in ARCHITECTURES[arch][1]
    model = load_model_dir(str(tmp_path / "ok"))
    assert isinstance(model, Nelovik) and isinstance(model, StreamDecoder) and model.ingest_stats["tensors"] == len(W)
    assert all(torch.equal(model.weights[k], W[k]) for k in W)
    missing = dict(W)
    missing.pop("l0.mix.left.sink")
    _write_checkpoint(tmp_path / "missing", cfg, missing)
    with pytest.raises(RuntimeError, match="Missing"):
        load_model_dir(str(tmp_path / "missing"))
    _write_checkpoint(tmp_path / "shape", cfg, dict(W, **{"l1.mix.q.conv": W["l1.mix.q.conv"][:, :-1].contiguous()}))
    with pytest.raises(RuntimeError, match="size mismatch"):
        load_model_dir(str(tmp_path / "shape"))
    with pytest.raises(NotImplementedError):
        load_model_dir(str(tmp_path / "ok"), dtype=torch.float16)


def test_model_refuses_to_run_without_cuda():
    from evo_b200 import _lib
    cfg = O.make_config()
    m = Nelovik(NelovikConfig.from_dict(cfg))
    m.load_state_dict(O.random_weights(cfg))
    with pytest.raises(RuntimeError):
        m.load_state_dict({"embed": torch.zeros(2, 2)})
    with pytest.raises(_lib.EvoError, match="no CPU"):
        m(torch.zeros(1, 4, dtype=torch.long))
    rnd = Nelovik(NelovikConfig.from_dict(cfg)).init_random(seed=3)
    assert set(rnd.weights) == set(O.tensor_shapes(cfg)) and all(torch.isfinite(v.float()).all() for v in rnd.weights.values())
    assert m.fir_taps == 3


def test_oracle_visibility_rotation_and_activation():
    # tokens: the last `window` positions; blocks: those that end at or before i - window
    assert O.visible_tokens(10, 4) == [7, 8, 9, 10] and O.visible_tokens(2, 4) == [0, 1, 2]
    assert O.visible_blocks(10, 4, 3) == [0, 1] and O.visible_blocks(11, 4, 3) == [0, 1] and O.visible_blocks(12, 4, 3) == [0, 1, 2]
    assert O.visible_blocks(5, 4, 3) == [] and O.visible_blocks(6, 4, 3) == [0] and O.visible_blocks(100, 4, 0) == []
    for i in range(40):                                   # a token is never seen twice, and the gap holds the tokens of the blocks not yet seen
        direct = set(O.visible_tokens(i, 6))
        pooled = {t for b in O.visible_blocks(i, 6, 4) for t in range(4 * b, 4 * b + 4)}
        assert not (direct & pooled) and max(pooled, default=-1) < min(direct)
        assert len(set(range(i + 1)) - direct - pooled) < 4
    # rotation: entry i pairs with entry i + dims/2; entries past dims pass; position 0 is the identity
    v = torch.arange(1.0, 7.0, dtype=torch.float64).view(1, 1, 6)
    assert torch.equal(O.rotate_half(v, torch.tensor([0]), 4, 50.0), v)
    r = O.rotate_half(v, torch.tensor([3]), 4, 50.0)[0, 0]
    a1 = 3 * 50.0 ** -0.5
    assert torch.allclose(r[[0, 2]], torch.tensor([math.cos(3.0) - 3 * math.sin(3.0), 3 * math.cos(3.0) + math.sin(3.0)], dtype=torch.float64))
    assert torch.allclose(r[[1, 3]], torch.tensor([2 * math.cos(a1) - 4 * math.sin(a1), 4 * math.cos(a1) + 2 * math.sin(a1)], dtype=torch.float64))
    assert torch.equal(r[4:], v[0, 0, 4:])
    # the activation is continuous with a continuous slope 1/2 at 0, quadratic above, bounded slope below
    p, q = torch.tensor(0.3, dtype=torch.float64), torch.tensor(0.8, dtype=torch.float64)
    z = torch.tensor([-1e-6, 0.0, 1e-6], dtype=torch.float64)
    y = O.xielu(z, p, q)
    assert y[1] == 0 and abs((y[2] - y[0]) / 2e-6 - 0.5) < 1e-5
    big = O.xielu(torch.tensor([3.0, -40.0], dtype=torch.float64), p, q)
    sp = lambda t: math.log1p(math.exp(t))
    assert math.isclose(big[0], sp(0.3) * 9 + 1.5) and math.isclose(big[1], (0.5 + sp(0.8)) * (math.exp(-40.0) - 1 + 40) - 20)


def test_delta_rule_read_out_sees_the_current_write():
    """o_t = S_t^T q_t with S_t already holding token t: with no decay and beta = 1, a query equal to the (unit) key returns the value
    just written, whatever came before along other directions."""
    dk, dv = 4, 3
    S = torch.zeros(dk, dv, dtype=torch.float64)
    k1, k2 = torch.tensor([1.0, 0, 0, 0], dtype=torch.float64), torch.tensor([0, 1.0, 0, 0], dtype=torch.float64)
    v1, v2 = torch.tensor([1.0, 2, 3], dtype=torch.float64), torch.tensor([-1.0, 0, 5], dtype=torch.float64)
    for k, v in ((k1, v1), (k2, v2), (k1, v2)):
        u = v - S.T @ k
        S = S + torch.outer(k, u)
        assert torch.allclose(S.T @ k, v)
    assert torch.allclose(S.T @ k2, v2)
    # the same step written from the decayed state alone: o = (gS)^T q + u (k . q)
    g, beta = 0.7, 0.4
    S0 = torch.randn(dk, dv, dtype=torch.float64)
    k, q, v = torch.randn(dk, dtype=torch.float64), torch.randn(dk, dtype=torch.float64), torch.randn(dv, dtype=torch.float64)
    Sd = g * S0
    u = beta * (v - Sd.T @ k)
    assert torch.allclose((Sd + torch.outer(k, u)).T @ q, Sd.T @ q + u * (k @ q))
