"""Movalorn on the GPU against the plain oracle (oracle/movalorn_oracle.py): every mechanism's kernel alone, then the model --
whole prompts, token-by-token decoding, portions down to two tokens, batches, reused cache memory, window edges in prompts and in
steps, the first tokens of a sequence, long decoding, other sizes -- and greedy generation through the framework's Generator and
command line.  Small configurations, random weights; where random weights would hide a fault the inputs are made so that it shows."""
import ctypes as C
import math

import pytest
import torch

from evo_b200 import _lib
from evo_b200._lib import BranchNormParams, MinGruParams, check, ptr
from oracle import movalorn_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F32, B16 = torch.float32, torch.bfloat16


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _bf(t):
    return t.to(B16)


def _close(got, want, tol, what=""):
    err = (got.double().cpu() - want.double().cpu()).abs().max().item()
    ref = max(want.abs().max().item(), 1e-6)
    assert err <= tol * ref, f"{what}: max err {err:.3e} vs scale {ref:.3e} (tol {tol})"


# ------------------------------------------------------------------ kernels alone
@pytest.mark.parametrize("ids_dtype", [torch.int64, torch.int32])
def test_pair_embedding_first_token_carried_token_and_batch(ids_dtype):
    V, D, n, a, b, scale = 37, 24, 11, 5, 3, 2.5
    g = torch.Generator().manual_seed(1)
    w = {"embed": _bf(torch.randn(V, D, generator=g)), "bigram": _bf(torch.randn(n + 1, D, generator=g))}
    emb = {"scale": scale, "bigram": {"buckets": n, "mul_prev": a, "mul_cur": b}}
    ids = torch.randint(0, V, (2, 9), generator=g)
    wd = {k: v.to(DEV) for k, v in w.items()}
    lib = _lib.lib()

    def run(part, prev):
        out = torch.empty(part.numel(), D, device=DEV)
        pd = part.to(DEV, ids_dtype).contiguous()
        check(lib.evo_embed_pair_f32(ptr(pd), int(ids_dtype == torch.int64), ptr(wd["embed"]), ptr(wd["bigram"]), ptr(out), ptr(prev),
                                     part.shape[0], part.shape[1], D, V, scale, n, a, b, _stream()))
        return out.view(part.shape[0], part.shape[1], D)

    want = torch.stack([O.embed_tokens(ids[r].tolist(), None, {k: v.double() for k, v in w.items()}, emb) for r in range(2)])
    _close(run(ids, None), want, 1e-6, "stateless")
    prev = torch.full((2,), -1, dtype=torch.int64, device=DEV)
    parts = [run(ids[:, :1], prev), run(ids[:, 1:3], prev), run(ids[:, 3:], prev)]
    _close(torch.cat(parts, 1), want, 1e-6, "carried previous token")
    assert prev.tolist() == ids[:, -1].tolist()


@pytest.mark.parametrize("D,ldo", [(96, 128), (130, 192), (1032, 1088), (4100, 4160)])
def test_branch_norm_modes(D, ldo):
    M, eps = 5, 1e-5
    g = torch.Generator().manual_seed(D)
    x = torch.randn(M, D, generator=g)
    y, gate = _bf(torch.randn(M, D + 8, generator=g)), _bf(torch.randn(M, D + 16, generator=g))
    gb, step = _bf(torch.randn(D, generator=g)), _bf(torch.randn(D, generator=g))
    x0 = torch.randn(M, D, generator=g)
    yd, gd, gbd, sd, x0d = (t.to(DEV) for t in (y, gate, gb, step, x0))
    lib = _lib.lib()
    u = y[:, :D].double() * torch.sigmoid(gate[:, :D].double() + gb.double())
    # gated, normed branch added to the stream, then the next norm
    xn = x.double() + O.scalar_norm(u, 0.7, eps)
    xb, outb = x.to(DEV), torch.full((M, ldo), 7.0, dtype=B16, device=DEV)                 # bf16 activations in and out
    pb = BranchNormParams(x=xb.data_ptr(), y=yd.data_ptr(), ldy=D + 8, gate=gd.data_ptr(), ldg=D + 16, gate_bias=gbd.data_ptr(), post_norm=1, post_gain=0.7,
                          gain=1.3, eps=eps, out=outb.data_ptr(), ldo=ldo, dtype=0, rows=M, D=D)
    check(lib.evo_branch_norm(C.byref(pb), _stream()))
    _close(xb, xn, 1e-6, "stream, bf16 branch")
    _close(outb[:, :D], O.scalar_norm(xn, 1.3, eps), 5e-3, "opened norm in bf16")
    assert (outb[:, D:] == 0).all()
    yf, gf = y.float().to(DEV), gate.float().to(DEV)
    xd, out = x.to(DEV), torch.full((M, ldo), 7.0, device=DEV)
    p = BranchNormParams(x=xd.data_ptr(), y=yf.data_ptr(), ldy=D + 8, gate=gf.data_ptr(), ldg=D + 16, gate_bias=gbd.data_ptr(), post_norm=1, post_gain=0.7,
                         gain=1.3, eps=eps, out=out.data_ptr(), ldo=ldo, dtype=1, rows=M, D=D)
    check(lib.evo_branch_norm(C.byref(p), _stream()))
    _close(xd, xn, 1e-6, "stream")
    _close(out[:, :D], O.scalar_norm(xn, 1.3, eps), 1e-6, "opened norm")
    assert (out[:, D:] == 0).all()
    # gathered rows: no write-back
    xd2, out2 = x.to(DEV), torch.full((2, ldo), 7.0, device=DEV)
    rows = torch.tensor([3, 1], device=DEV)
    p.x, p.out, p.rows, p.gather = xd2.data_ptr(), out2.data_ptr(), 2, rows.data_ptr()
    check(lib.evo_branch_norm(C.byref(p), _stream()))
    _close(out2[:, :D], O.scalar_norm(xn[[3, 1]], 1.3, eps), 1e-6, "gathered rows")
    assert torch.equal(xd2.cpu(), x)
    # replace: the stream becomes the branch plus a row vector; fp32 activations
    xd3, out3 = x.to(DEV), torch.full((M, ldo), 7.0, device=DEV)
    p3 = BranchNormParams(x=xd3.data_ptr(), y=yf.data_ptr(), ldy=D + 8, replace=1, row_add=sd.data_ptr(), gain=0.9, eps=eps, out=out3.data_ptr(), ldo=ldo,
                          dtype=1, rows=M, D=D)
    check(lib.evo_branch_norm(C.byref(p3), _stream()))
    xr = y[:, :D].double() + step.double()
    _close(xd3, xr, 1e-6, "replaced stream")
    _close(out3[:, :D], O.scalar_norm(xr, 0.9, eps), 1e-6, "norm after replace")
    # concat: pending branch folded, [x | x0] cast, no norm
    ld2 = 2 * D + 24
    xd4, out4 = x.to(DEV), torch.full((M, ld2), 7.0, device=DEV)
    p4 = BranchNormParams(x=xd4.data_ptr(), y=yf.data_ptr(), ldy=D + 8, gain=1.0, eps=eps, out=out4.data_ptr(), ldo=ld2, concat=1, cat=x0d.data_ptr(), dtype=1, rows=M, D=D)
    check(lib.evo_branch_norm(C.byref(p4), _stream()))
    _close(out4[:, :D], x.double() + y[:, :D].double(), 1e-6, "concat left")
    _close(out4[:, D:2 * D], x0.double(), 0, "concat right")
    assert (out4[:, 2 * D:] == 0).all()
    # nothing pending, no output: the stream stays
    p5 = BranchNormParams(x=xd4.data_ptr(), gain=1.0, eps=eps, dtype=1, rows=M, D=D)
    before = xd4.clone()
    check(lib.evo_branch_norm(C.byref(p5), _stream()))
    assert torch.equal(before, xd4)


@pytest.mark.parametrize("act", [0, 1])
def test_glu_activation_with_group_weights_and_scaled_logits(act):
    M, F, grp, E = 4, 52, 9, 4                         # 4 weighted groups of 9 columns, 16 unweighted columns after them
    g = torch.Generator().manual_seed(act)
    z = torch.randn(M, 2 * F + 3, generator=g) * 2
    wts = torch.rand(M, E, generator=g)
    wts[0, 1] = 0.0
    zd, wd, out = z.to(DEV), wts.to(DEV), torch.full((M, F + 12), 3.0, device=DEV)
    lib = _lib.lib()
    check(lib.evo_glu_act(ptr(zd), C.c_void_p(zd.data_ptr() + 4 * F), 2 * F + 3, ptr(out), F + 12, M, F, act, ptr(wd), E, grp, E, 0, 1, _stream()))
    fn = O.gelu_tanh if act == 0 else O.silu
    want = fn(z[:, :F].double()) * z[:, F:2 * F].double()
    for e in range(E):
        want[:, e * grp:(e + 1) * grp] *= wts[:, e:e + 1].double()
    _close(out[:, :F], want, 2e-6, "glu")
    assert (out[:, F:] == 0).all()
    check(lib.evo_glu_act(ptr(zd), C.c_void_p(zd.data_ptr() + 4 * F), 2 * F + 3, ptr(out), F + 12, M, F, act, None, 0, 0, 0, 0, 1, _stream()))
    _close(out[:, :F], fn(z[:, :F].double()) * z[:, F:2 * F].double(), 2e-6, "glu without weights")
    scaled = torch.empty(M, F, device=DEV)
    check(lib.evo_scale_logits(ptr(zd), 2 * F + 3, ptr(scaled), M, F, 0.37, 1, _stream()))
    _close(scaled, z[:, :F].double() * 0.37, 1e-6, "logit scale")


@pytest.mark.parametrize("W,T", [(40, 50), (130, 300), (257, 129)])
@pytest.mark.parametrize("dtype", [F32, B16])
def test_mingru_whole_portions_and_steps(W, T, dtype):
    """whole sequence (chunked scan above 128 tokens) == portions through the carried state == the oracle's token loop."""
    B, ld, ldo = 2, 3 * W + 5, W + 7
    g = torch.Generator().manual_seed(W)
    z = torch.randn(B, T, ld, generator=g).to(dtype)
    bz, bu = _bf(torch.randn(W, generator=g)), _bf(torch.randn(W, generator=g))
    zf = z.double()
    S = torch.zeros(B, W, dtype=torch.float64)
    want = torch.empty(B, T, W, dtype=torch.float64)
    for t in range(T):
        a = torch.sigmoid(zf[:, t, :W] + bz.double())
        c = zf[:, t, W:2 * W] + bu.double()
        S = (1 - a) * S + a * torch.where(c >= 0, c + 0.5, torch.sigmoid(c))
        want[:, t] = S * O.silu(zf[:, t, 2 * W:3 * W])
    bzd, bud = bz.to(DEV), bu.to(DEV)
    lib = _lib.lib()
    esz = z.element_size()

    def run(lo, hi, state, zero):
        part = z[:, lo:hi].contiguous().to(DEV)
        out = torch.full((B, hi - lo, ldo), 9.0, dtype=dtype, device=DEV)
        p = MinGruParams(z=part.data_ptr(), u=part.data_ptr() + W * esz, g=part.data_ptr() + 2 * W * esz, ld=ld, z_bias=bzd.data_ptr(), u_bias=bud.data_ptr(),
                         state=state.data_ptr() if state is not None else None, zero_start=zero, out=out.data_ptr(), ldo=ldo, dtype=int(dtype == F32), B=B, L=hi - lo, W=W)
        n = lib.evo_mingru_workspace(C.byref(p))
        ws = torch.empty(max(n, 1), dtype=torch.uint8, device=DEV)
        check(lib.evo_mingru_fwd(C.byref(p), ptr(ws), n, _stream()))
        assert (out[:, :, W:] == 0).all()
        return out[:, :, :W]

    tol = 2e-5 if dtype == F32 else 1e-2
    _close(run(0, T, None, 1), want, tol, "whole, no state")
    state = torch.full((B, W), float("nan"), device=DEV)
    cuts = [0, 1, 3, 5, 5 + 140, T - 1, T] if T > 160 else [0, 2, 3, T - 20, T - 19, T]
    outs = [run(cuts[i], cuts[i + 1], state, int(i == 0)) for i in range(len(cuts) - 1)]
    _close(torch.cat(outs, 1), want, tol, "portions through the state")
    _close(state, S, 2e-5, "final state")


@pytest.mark.parametrize("E,top,D,M", [(5, 2, 48, 9), (16, 4, 100, 1100), (40, 1, 64, 1030), (3, 3, 33, 9), (70, 6, 36, 17)])
def test_router_scores_choice_and_weights(E, top, D, M):
    scale = 1.7
    g = torch.Generator().manual_seed(E)
    h = torch.randn(M, D + 3, generator=g)
    rw, corr = _bf(torch.randn(E, D, generator=g) * 0.5), _bf(torch.randn(E, generator=g) * 0.4)
    hd, rwd, cd = h.to(DEV), rw.to(DEV), corr.to(DEV)
    wts, chosen = torch.full((M, E), 5.0, device=DEV), torch.zeros(M, top, dtype=torch.int32, device=DEV)
    check(_lib.lib().evo_moe_route(ptr(hd), D + 3, ptr(rwd), ptr(cd), ptr(wts), ptr(chosen), M, D, E, top, scale, 1, _stream()))
    s = torch.softmax(h[:, :D].double() @ rw.double().T, -1)
    pick = torch.topk(s + corr.double(), top).indices
    want = torch.zeros(M, E, dtype=torch.float64)
    want.scatter_(1, pick, s.gather(1, pick) * scale)
    _close(wts, want, 1e-5, "routing weights")
    assert sorted(map(tuple, chosen.cpu().sort(1).values.tolist())) == sorted(map(tuple, pick.sort(1).values.tolist()))
    # the correction changes the choice, not the weight: a large correction on the weakest expert selects it with its own score
    worst = int(s[0].argmin())
    corr2 = corr.clone()
    corr2[worst] = 10.0
    check(_lib.lib().evo_moe_route(ptr(hd), D + 3, ptr(rwd), ptr(corr2.to(DEV)), ptr(wts), None, M, D, E, top, scale, 1, _stream()))
    assert abs(wts[0, worst].item() - s[0, worst].item() * scale) < 1e-6


# ------------------------------------------------------------------ the model
def _model(cfg, W, dtype=F32):
    from evo_b200.movalorn import Movalorn, MovalornConfig
    m = Movalorn(MovalornConfig.from_dict(cfg), dtype=dtype)
    m.load_state_dict(W)
    return m.to(DEV)


def _portions(model, tokens, sizes, max_seqlen=None, state=None):
    state = state or model.initialize_inference_params(max_seqlen=max_seqlen or len(tokens) + 8, max_batch_size=1)
    outs, t = [], 0
    for n in sizes:
        state["mha"].seqlen_offset = state["hyena"].seqlen_offset = t
        lg, _ = model(torch.tensor([tokens[t:t + n]], device=DEV), inference_params_dict=state)
        outs.append(lg[0])
        t += n
    assert t == len(tokens)
    return torch.cat(outs, 0)


@pytest.mark.parametrize("mode", ["prompt", "portions", "steps", "steps_per_head"])
@pytest.mark.parametrize("H,dim,rd,vd,rank,window", [(3, 8, 4, 10, 12, 7), (1, 16, 8, 16, 40, 33), (2, 24, 2, 6, 9, 600), (5, 4, 12, 36, 130, 2), (13, 8, 6, 8, 70, 50),
                                                     (9, 8, 4, 8, 600, 21)])
def test_latent_attention_mixer_matches_the_oracle(mode, H, dim, rd, vd, rank, window):
    """The mixer alone (input rows -> projections -> cache -> attention -> output projection) against the oracle's token loop:
    the absorbed kernel (steps, short portions) and the expanded path (prompts) compute the same function."""
    cfg = O.make_config(layers=("latent_attention",), heads=H, dim=dim, rot_dim=rd, vdim=vd, kv_rank=rank, window=window, width=64)
    W = O.random_weights(cfg, seed=H * window)
    model = _model(cfg, W)
    model._ensure_packed()
    T = 70 if window < 100 else 660
    g = torch.Generator().manual_seed(3)
    h = torch.randn(T, 64, generator=g)
    m = cfg["layers"][0]["mixer"]
    rows = None if T < 100 else list(range(0, T, 37)) + [T - 1, window - 1, window, window + 1]
    want = O.latent_attention(h.double(), {k: v.double() for k, v in W.items()}, "l0.mix.", m, cfg["norm"]["eps"], [], rows=rows)
    hd = h.to(DEV)
    mc = model.config.layers[0].mixer
    state = model.initialize_inference_params(max_seqlen=T, max_batch_size=1)
    sizes = {"prompt": [T], "portions": [5, 2, 30, 3, T - 40], "steps": [T - 20] + [1] * 20, "steps_per_head": [T - 24] + [1] * 20 + [4]}[mode]
    if mode == "steps_per_head":
        model.latent_decode_path = "head"
    outs, t = [], 0
    with torch.no_grad():
        for n in sizes:
            pend = model._latent_attention(0, 0, mc, hd[t:t + n].contiguous(), 1, n, state["mha"], t, None)
            outs.append(pend.y[:, :64].clone())
            t += n
    got = torch.cat(outs, 0)
    if rows is not None:
        got, want = got[rows], want[rows]
    _close(got, want, 2e-5, f"{mode}")


@pytest.mark.parametrize("H,dim,rd,vd,rank,window,B", [(16, 16, 16, 24, 64, 150, 1), (13, 8, 32, 8, 128, 70, 3), (20, 8, 16, 16, 256, 300, 2)])
def test_latent_attention_steps_on_tensor_cores(H, dim, rd, vd, rank, window, B):
    """bf16 activations, groups of 16 heads, latents of 64 / 128 / 256 entries: the step attention runs its scores and value sums on the
    tensor cores.  Same inputs through the per-(query, head) kernel (fp32 arithmetic throughout) must agree to the output's bf16 rounding,
    and both with the oracle to bf16 accuracy; steps start inside the first tile, cross tile borders and run past the window."""
    cfg = O.make_config(layers=("latent_attention",), heads=H, dim=dim, rot_dim=rd, vdim=vd, kv_rank=rank, window=window, width=64)
    W = O.random_weights(cfg, seed=rank)
    model = _model(cfg, W, B16)
    model._ensure_packed()
    T0, steps = 40, 2 * window // 3 + 70
    T = T0 + steps
    h = _bf(torch.randn(B, T, 64, generator=torch.Generator().manual_seed(4)))
    m = cfg["layers"][0]["mixer"]
    rows = sorted(set(list(range(T0, T, 23)) + [T0, T0 + 1, 63, 64, 65, 127, 128, window - 1, window, window + 1, T - 1]) & set(range(T0, T)))
    want = O.latent_attention(h[0].double(), {k: v.double() for k, v in W.items()}, "l0.mix.", m, cfg["norm"]["eps"], [], rows=rows)[rows]
    hd = h.to(DEV)
    mc = model.config.layers[0].mixer
    outs = {}
    for path in ("shared", "head"):
        model.latent_decode_path = path
        state = model.initialize_inference_params(max_seqlen=T + 5, max_batch_size=B)
        got = []
        with torch.no_grad():
            model._latent_attention(0, 0, mc, hd[:, :T0].reshape(B * T0, 64).contiguous(), B, T0, state["mha"], 0, None)
            for t in range(T0, T):
                pend = model._latent_attention(0, 0, mc, hd[:, t].contiguous(), B, 1, state["mha"], t, None)
                got.append(pend.y[:, :64].float().clone())
        outs[path] = torch.stack(got, 1)                      # (B, steps, 64)
    _close(outs["shared"], outs["head"], 1.2e-2, "tensor-core steps against the fp32 per-head kernel")
    idx = [r - T0 for r in rows]
    _close(outs["shared"][0, idx], want, 2.5e-2, "tensor-core steps against the oracle")
    _close(outs["head"][0, idx], want, 2.5e-2, "per-head steps against the oracle")


def _dominant_token_weights(cfg, W, plain, odd):
    """Weights under which the key of the token `odd` (after `plain`) beats a plain key by 10 in every head, whatever the distance:
    the rotated query rows are zeroed (scores no longer depend on the position) and every head's unrotated query rows are scaled."""
    m = cfg["layers"][0]["mixer"]
    H, dim, rd, rank = m["heads"], m["dim"], m["rot_dim"], m["kv_rank"]
    w = {k: v.double() for k, v in W.items()}
    x = O.embed_tokens([plain, plain, odd], None, w, cfg["embedding"])
    h = O.scalar_norm(x, w["l0.norm1"], cfg["norm"]["eps"])
    lat = lambda row: O.rms((w["l0.mix.dkv"] @ row)[:rank], cfg["norm"]["eps"]) * w["l0.mix.dkv.norm"]
    dc = lat(h[2]) - lat(h[1])
    q = (w["l0.mix.q"] @ h[1]).view(H, dim + rd)
    out = dict(W)
    wq = W["l0.mix.q"].double().view(H, dim + rd, -1).clone()
    for hd in range(H):
        delta = float(q[hd, :dim] @ (w["l0.mix.uk"][hd * dim:(hd + 1) * dim] @ dc)) * m["scale"]
        wq[hd, :dim] *= 10.0 / delta
        wq[hd, dim:] = 0.0
    out["l0.mix.q"] = wq.view(H * (dim + rd), -1).to(B16)
    return out


@pytest.mark.parametrize("dtype", [F32, B16])
@pytest.mark.parametrize("window", [5, 40, 530])
def test_window_edge_with_one_dominant_token(dtype, window):
    """A one-layer attention model over a prompt of equal tokens with one other token at position j whose key dominates every softmax
    that sees it.  Position j + window - 1 is the last one that sees it; rows j and j + 1 of the stream differ from the rest (the pair
    embedding sees the other token twice), so from position j + 1 + window on the logits equal those of the plain prompt -- in a
    prompt, in portions that cut the window, and in single steps."""
    cfg = O.make_config(layers=("latent_attention",), window=window, heads=2, dim=16, rot_dim=8, vdim=16, kv_rank=24, width=64, vocab=50, no_ff_layers=(0,))
    W = _dominant_token_weights(cfg, O.random_weights(cfg, seed=window), 7, 31)
    model = _model(cfg, W, dtype)
    j = 9
    T = j + window + 6
    plain, odd = [7] * T, [7] * T
    odd[j] = 31
    base, _ = model(torch.tensor([plain], device=DEV))
    tol_same, tol_diff = (1e-5, 0.1) if dtype == F32 else (2e-2, 0.1)
    scale = base.abs().max().item()
    last_in, first_out = j + window - 1, j + 1 + window
    want = O.forward(cfg, W, odd) if (dtype == F32 and window < 100) else None
    for name, sizes in (("prompt", [T]), ("portions", [j + 1, 2, window - 3, 2, 2, T - j - window - 4]), ("steps", [j + 2] + [1] * (T - j - 2))):
        got = _portions(model, odd, sizes)
        d = (got - base[0]).abs().max(-1).values / scale
        assert d[last_in] > tol_diff, f"{name}: the token at the window's inner edge is not seen ({d[last_in]:.2e})"
        assert d[first_out:].max() < tol_same, f"{name}: a token outside the window is seen ({d[first_out:].max():.2e})"
        if want is not None:
            _close(got, want, 2e-5, name)


CONFIGS = {
    "mixed": dict(layers=("mingru", "mingru", "latent_attention"), moe_layers=(1, 2), loop=(1, 3, 2)),
    "loop_from_0": dict(layers=("latent_attention", "mingru"), loop=(0, 1, 3), moe_layers=(0,), top=1, experts=3, shared_ff=0, window=4, width=72, vocab=257,
                        logit_scale=1.0, embed_scale=1.0),
    "no_loop_no_ff": dict(layers=("mingru", "latent_attention", "latent_attention"), no_ff_layers=(0, 2), heads=2, dim=16, rot_dim=16, vdim=16, kv_rank=16,
                          gru_width=48, window=6, mul_prev=1, mul_cur=1, buckets=7),
    "wide": dict(layers=("mingru", "latent_attention"), loop=(0, 2, 2), moe_layers=(0, 1), experts=9, top=9, expert_ff=40, shared_ff=8, heads=1, dim=72,
                 rot_dim=32, vdim=136, kv_rank=200, gru_width=300, width=200, ff=264, window=1000),
}


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_model_whole_steps_and_portions_match_the_oracle_in_fp32(name):
    cfg = O.make_config(**CONFIGS[name])
    W = O.random_weights(cfg, seed=len(name))
    T = 75
    tokens = torch.randint(0, cfg["vocab"], (T,), generator=torch.Generator().manual_seed(1)).tolist()
    streams = []
    want = O.forward(cfg, W, tokens, tap=streams)
    model = _model(cfg, W)
    model._tap = []
    got, _ = model(torch.tensor([tokens], device=DEV))
    for r, (a, b) in enumerate(zip(model._tap, streams)):
        _close(a, b, 2e-5, f"{name}: residual stream after run {r}")
    assert len(model._tap) == len(streams)
    model._tap = None
    _close(got[0], want, 2e-5, f"{name}: whole")
    _close(_portions(model, tokens, [1] * T), want, 2e-5, f"{name}: token by token from the first token")
    _close(_portions(model, tokens, [40] + [1] * 35), want, 2e-5, f"{name}: prompt then steps")
    _close(_portions(model, tokens, [2, 2, 3, 30, 1, 2, 17, 9, 2, 5, 2]), want, 2e-5, f"{name}: portions")
    model.moe_sparse_min_rows = 2                      # expert layers run only the chosen experts (the prompt path), steps stay dense
    sparse, _ = model(torch.tensor([tokens], device=DEV))
    _close(sparse[0], want, 2e-5, f"{name}: whole, sparse experts")
    _close(_portions(model, tokens, [2, 2, 3, 30, 1, 2, 17, 9, 2, 5, 2]), want, 2e-5, f"{name}: portions, sparse experts")
    model.moe_sparse_min_rows = 1024
    _close(_portions(model, tokens[:1], [1]), want[:1], 2e-5, f"{name}: a one-token sequence")
    _close(_portions(model, tokens[:2], [2]), want[:2], 2e-5, f"{name}: a two-token sequence")


def test_layers_with_their_own_sizes_and_a_cache_that_has_to_grow():
    cfg = O.make_config(layers=("latent_attention", "mingru", "latent_attention", "mingru"), loop=(1, 3, 2), width=104, vocab=211, moe_layers=(2,))
    cfg["layers"][2]["mixer"] = {"heads": 4, "dim": 8, "rot_dim": 6, "vdim": 40, "kv_rank": 20, "scale": 0.2, "mask": {"size": 3}, "rot": {"base": 7.0, "dims": 6}}
    cfg["layers"][3]["mixer"] = {"width": 24}
    cfg["layers"][1]["mlp"] = None
    cfg["layers"][3]["mlp"]["ff"] = 72
    W = O.random_weights(cfg, seed=21)
    tokens = torch.randint(0, cfg["vocab"], (70,), generator=torch.Generator().manual_seed(8)).tolist()
    want = O.forward(cfg, W, tokens)
    model = _model(cfg, W)
    got, _ = model(torch.tensor([tokens], device=DEV))
    _close(got[0], want, 2e-5, "whole")
    state = model.initialize_inference_params(max_seqlen=16, max_batch_size=1)
    _close(_portions(model, tokens, [9, 2, 20, 1, 1, 30, 7], state=state), want, 2e-5, "portions through a growing cache")
    assert all(c.shape[1] >= 70 for c in state["mha"].key_value_memory_dict.values())


def test_model_bf16_stays_within_rounding_of_the_oracle_and_of_itself():
    cfg = O.make_config(**CONFIGS["mixed"])
    W = O.random_weights(cfg, seed=3)
    tokens = torch.randint(0, cfg["vocab"], (90,), generator=torch.Generator().manual_seed(2)).tolist()
    want = O.forward(cfg, W, tokens)
    model = _model(cfg, W, B16)
    whole, _ = model(torch.tensor([tokens], device=DEV))
    cut = _portions(model, tokens, [50, 2, 1, 1, 30, 6])
    rel = lambda a, b: ((a.double().cpu() - b.double().cpu()).pow(2).mean().sqrt() / b.double().pow(2).mean().sqrt()).item()
    assert rel(whole[0], want) < 3e-2
    assert rel(cut, want) < 3e-2
    assert rel(cut, whole[0].cpu()) < 3e-2
    model.moe_sparse_min_rows = 2
    sparse, _ = model(torch.tensor([tokens], device=DEV))
    assert rel(sparse[0], want) < 3e-2 and rel(sparse[0], whole[0].cpu()) < 3e-2
    model.moe_sparse_min_rows = 1024
    model.gemm_path = "simt"                              # the tensor-core linear layers against the CUDA-core ones
    simt, _ = model(torch.tensor([tokens], device=DEV))
    assert rel(simt[0], whole[0].cpu()) < 2e-2


def test_batch_rows_equal_each_sequence_alone_and_wanted_rows_select():
    cfg = O.make_config(**CONFIGS["mixed"])
    W = O.random_weights(cfg, seed=5)
    model = _model(cfg, W)
    ids = torch.randint(0, cfg["vocab"], (3, 33), generator=torch.Generator().manual_seed(4)).to(DEV)
    both, _ = model(ids)
    for b in range(3):
        alone, _ = model(ids[b:b + 1])
        _close(both[b], alone[0].double().cpu(), 1e-6, f"row {b}")
    state = model.initialize_inference_params(max_seqlen=64, max_batch_size=3)
    a, _ = model(ids[:, :20], inference_params_dict=state)
    state["mha"].seqlen_offset = 20
    b_, _ = model(ids[:, 20:], inference_params_dict=state)
    _close(torch.cat([a, b_], 1), both.double().cpu(), 1e-5, "batched portions")
    rows = [0, 7, 32, 40, 98]
    picked, _ = model(ids, logits_rows=rows)
    _close(picked, both.reshape(-1, both.shape[-1])[rows].double().cpu(), 1e-6, "wanted rows")


def test_reused_cache_memory_and_long_decoding_past_the_window():
    """A cache that still holds another request's rows (and NaNs beyond) serves a new request; decoding runs far past the window;
    a request interleaved with another one keeps its own state."""
    cfg = O.make_config(**dict(CONFIGS["mixed"], window=11))
    W = O.random_weights(cfg, seed=7)
    model = _model(cfg, W)
    g = torch.Generator().manual_seed(6)
    a = torch.randint(0, cfg["vocab"], (120,), generator=g).tolist()
    b = torch.randint(0, cfg["vocab"], (60,), generator=g).tolist()
    want_a, want_b = O.forward(cfg, W, a), O.forward(cfg, W, b)
    state = model.initialize_inference_params(max_seqlen=128, max_batch_size=1)
    _close(_portions(model, a, [20] + [1] * 100, state=state), want_a, 2e-5, "long decoding")
    for cache in state["mha"].key_value_memory_dict.values():
        cache[:, 100:, :12] = float("nan")
    reused = model.initialize_inference_params(max_seqlen=128, max_batch_size=1)
    reused["mha"].key_value_memory_dict = state["mha"].key_value_memory_dict           # same memory, stale contents
    _close(_portions(model, b, [7, 2, 51], state=reused), want_b, 2e-5, "reused cache memory")
    sa = model.initialize_inference_params(max_seqlen=128, max_batch_size=1)
    sb = model.initialize_inference_params(max_seqlen=128, max_batch_size=1)
    outs_a, outs_b = [], []
    for lo, hi in ((0, 30), (30, 31), (31, 60)):
        for tokens, st, outs in ((a, sa, outs_a), (b, sb, outs_b)):
            st["mha"].seqlen_offset = lo
            lg, _ = model(torch.tensor([tokens[lo:hi]], device=DEV), inference_params_dict=st)
            outs.append(lg[0])
    _close(torch.cat(outs_a), want_a[:60], 2e-5, "interleaved a")
    _close(torch.cat(outs_b), want_b[:60], 2e-5, "interleaved b")


@pytest.mark.parametrize("device_loop", [True, False])
def test_greedy_generation_through_the_generator(device_loop):
    from evo_b200 import CharLevelTokenizer, Generator
    cfg = O.make_config(**dict(CONFIGS["mixed"], vocab=512))
    W = O.random_weights(cfg, seed=11)
    model = _model(cfg, W)
    gen = Generator(model, CharLevelTokenizer(512), top_k=1, top_p=1.0, temperature=1.0)
    gen.device_loop = device_loop
    prompt = torch.randint(0, 512, (1, 21), generator=torch.Generator().manual_seed(8)).to(DEV)
    n_new = 24
    picked, logits, _ = gen.generate(DEV, input_ids=prompt, num_tokens=n_new, cached_generation=True, force_prompt_threshold=64, print_generation=False, stop_at_eos=False)
    assert picked.shape == (1, n_new) and logits.shape == (1, n_new, 512)
    full = prompt[0].tolist() + picked[0].tolist()
    want = O.forward(cfg, W, full)
    for s in range(n_new):                                    # each picked token is (within rounding) the oracle's argmax given the same prefix
        row = want[len(full) - n_new - 1 + s]
        assert row[picked[0, s]] >= row.max() - 2e-2, s
        _close(logits[0, s], row, 2e-5 if not device_loop else 1e-2, f"kept logits {s}")     # the device loop keeps the sampler's bf16 view of the logits


def test_command_line_generates_and_replays_from_a_checkpoint_folder(tmp_path):
    """scripts/generate.py --model-dir and bin/trace_run: config.json picks the model class, the streaming loader fills it."""
    import json
    import os
    import subprocess
    import sys
    import numpy as np
    from tests.test_zaverax_host import ROOT, _write_checkpoint
    from scripts import generate as cli
    cfg = O.make_config(**dict(CONFIGS["mixed"], vocab=512))
    W = O.random_weights(cfg, seed=13)
    ckpt = str(tmp_path / "ckpt")
    _write_checkpoint(ckpt, cfg, W)
    texts, scores = cli.main(["--model-dir", ckpt, "--prompt", "ACGTTGCA", "--n-samples", "2", "--n-tokens", "9", "--top-k", "1", "--device", DEV, "--verbose", "0"])
    assert len(texts) == 2 and texts[0] == texts[1] and len(scores) == 2
    tokens = torch.randint(0, 512, (40,), generator=torch.Generator().manual_seed(5)).tolist()
    want = O.forward(cfg, W, tokens)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": tokens[:25], "want": [0, 24]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": tokens[25:27], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": tokens[27:28], "want": [0]}], "end": []},
             {"step": 3, "entries": [{"id": "a", "tokens": tokens[28:], "want": [11]}], "end": ["a"]},
             {"step": 4, "entries": [{"id": "b", "tokens": tokens[:3], "want": [2]}], "end": ["b"]}]
    out = str(tmp_path / "out")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", ckpt, "--dtype", "float32", "--out", out, "--max-tokens", "64"],
                       input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(5)]
    assert not os.path.exists(os.path.join(out, "1.f32"))
    for step, rows in ((0, [0, 24]), (2, [27]), (3, [39]), (4, [2])):
        got = torch.from_numpy(np.fromfile(os.path.join(out, f"{step}.f32"), dtype="<f4").reshape(len(rows), 512).copy())
        _close(got, want[rows], 2e-5, f"replayed step {step}")
