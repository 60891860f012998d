"""Nelovik on the GPU against the plain oracle (oracle/nelovik_oracle.py): the row kernels alone, every mixer alone over several
sizes, then the model -- whole prompts, token-by-token decoding, portions down to two tokens, batches, reused state memory, window
and pooled-block edges in prompts and in steps, far keys, the first tokens of a sequence, long decoding, other sizes -- and greedy
generation through the framework's Generator and command line.  Small configurations, random weights; where random weights would
hide a fault the weights are made so that it shows."""
import ctypes as C
import math

import pytest
import torch

from evo_b200 import _lib
from evo_b200._lib import ConvActParams, SumNormParams, check, ptr
from oracle import nelovik_oracle as O

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


def _model(cfg, W, dtype=F32):
    from evo_b200.nelovik import Nelovik, NelovikConfig
    m = Nelovik(NelovikConfig.from_dict(cfg), dtype=dtype)
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


def _tokens(cfg, n, seed=1):
    return torch.randint(0, cfg["vocab"], (n,), generator=torch.Generator().manual_seed(seed)).tolist()


# ------------------------------------------------------------------ kernels alone
@pytest.mark.parametrize("D,ldo", [(48, 64), (130, 192), (1032, 1088), (4100, 4160)])
@pytest.mark.parametrize("dtype", [F32, B16])
def test_sum_norm_branches_norms_and_gathered_rows(D, ldo, dtype):
    M, eps = 6, 1e-5
    g = torch.Generator().manual_seed(D)
    x = torch.randn(M, D, generator=g)
    ys = [_bf(torch.randn(M, D + 8 * b, generator=g)) for b in range(3)]
    nws = [_bf(1 + 0.3 * torch.randn(D, generator=g)), _bf(1 + 0.3 * torch.randn(D, generator=g)), None]
    scales = [0.5, 0.5, 1.0]
    w1, w2 = _bf(torch.randn(D, generator=g)), _bf(torch.randn(D, generator=g))
    xn = x.double()
    for y, nw, s in zip(ys, nws, scales):
        yy = y[:, :D].double()
        xn = xn + s * (O.rms(yy, eps) * nw.double() if nw is not None else yy)
    dt = 1 if dtype == F32 else 0
    tol = 1e-6 if dtype == F32 else 6e-3
    yd = [y.to(DEV, dtype) for y in ys]
    nwd = [n.to(DEV) if n is not None else None for n in nws]
    w1d, w2d = w1.to(DEV), w2.to(DEV)
    lib = _lib.lib()

    def params(xd, outs, rows, gather=None, nb=3):
        p = SumNormParams(x=xd.data_ptr(), n_branches=nb, eps=eps, dtype=dt, rows=rows, D=D, ldo=ldo, gather=gather.data_ptr() if gather is not None else None)
        for b in range(nb):
            p.y[b], p.ldy[b], p.norm_w[b], p.scale[b] = yd[b].data_ptr(), D + 8 * b, (nwd[b].data_ptr() if nwd[b] is not None else None), scales[b]
        for n, (o, w) in enumerate(outs):
            p.out[n], p.w[n] = o.data_ptr(), w.data_ptr()
        return p
    xd = x.to(DEV)
    o1, o2 = torch.full((M, ldo), 7.0, dtype=dtype, device=DEV), torch.full((M, ldo), 7.0, dtype=dtype, device=DEV)
    check(lib.evo_sum_norm(C.byref(params(xd, [(o1, w1d), (o2, w2d)], M)), _stream()))
    _close(xd, xn, 1e-6, "stream")
    _close(o1[:, :D], O.rms(xn, eps) * w1.double(), tol, "first norm")
    _close(o2[:, :D], O.rms(xn, eps) * w2.double(), tol, "second norm")
    assert (o1[:, D:] == 0).all() and (o2[:, D:] == 0).all()
    # gathered rows: the branches are added for the output only, the stream stays
    xd2, o3 = x.to(DEV), torch.full((2, ldo), 7.0, dtype=dtype, device=DEV)
    rows = torch.tensor([4, 1], device=DEV)
    check(lib.evo_sum_norm(C.byref(params(xd2, [(o3, w2d)], 2, gather=rows)), _stream()))
    _close(o3[:, :D], (O.rms(xn, eps) * w2.double())[[4, 1]], tol, "gathered rows")
    assert torch.equal(xd2.cpu(), x)
    # no branch: norms of the stream as it is; no output: only the sum
    xd3, o4 = x.to(DEV), torch.full((M, ldo), 7.0, dtype=dtype, device=DEV)
    check(lib.evo_sum_norm(C.byref(params(xd3, [(o4, w1d)], M, nb=0)), _stream()))
    _close(o4[:, :D], O.rms(x.double(), eps) * w1.double(), tol, "norm without branches")
    assert torch.equal(xd3.cpu(), x)
    check(lib.evo_sum_norm(C.byref(params(xd3, [], M, nb=1)), _stream()))
    _close(xd3, x.double() + 0.5 * O.rms(ys[0][:, :D].double(), eps) * nws[0].double(), 1e-6, "sum only")


@pytest.mark.parametrize("taps,Cn,L", [(4, 72, 90), (2, 5, 33), (1, 40, 12), (3, 300, 17), (8, 33, 70), (4, 70, 50)])
@pytest.mark.parametrize("dtype", [F32, B16])
def test_short_convolution_whole_portions_and_steps(taps, Cn, L, dtype):
    B, ld, col0 = 2, Cn + 24, 8
    g = torch.Generator().manual_seed(taps * L)
    src = _bf(torch.randn(B, L, ld, generator=g))
    w, bias = _bf(torch.randn(Cn, taps, generator=g)), _bf(torch.randn(Cn, generator=g))
    want = torch.stack([O.silu(O.short_conv(src[b, :, col0:col0 + Cn].double(), w.double(), bias.double())) for b in range(B)])
    wd, bd = w.to(DEV), bias.to(DEV)
    lib = _lib.lib()
    dt = 1 if dtype == F32 else 0

    def run(sizes, with_bias=True):
        carry = torch.full((B, max(taps - 1, 1), Cn), float("nan"), device=DEV)
        outs, t = [], 0
        for n in sizes:
            part = src[:, t:t + n].to(DEV, dtype).contiguous()
            out = torch.empty(B * n, Cn, dtype=dtype, device=DEV)
            p = ConvActParams(inp=part.data_ptr() + col0 * part.element_size(), ld=ld, weight=wd.data_ptr(), bias=bd.data_ptr() if with_bias else None,
                              carry=carry.data_ptr() if taps > 1 else None, zero_start=int(t == 0), out=out.data_ptr(), ldo=Cn,
                              B=B, L=n, C=Cn, taps=taps, act=1, dtype=dt)
            check(lib.evo_conv_act(C.byref(p), _stream()))
            outs.append(out.view(B, n, Cn))
            t += n
        assert t == L
        return torch.cat(outs, 1)
    tol = 1e-6 if dtype == F32 else 6e-3
    _close(run([L]), want, tol, "whole")
    _close(run([1] * L), want, tol, "steps")
    _close(run([2, 1, 2, L - 9, 3, 1]), want, tol, "portions")
    if L > 25:
        _close(run([L - 20, 17, 3]), want, tol, "portions longer than one thread's rows")
    nb = torch.stack([O.silu(O.short_conv(src[b, :, col0:col0 + Cn].double(), w.double())) for b in range(B)])
    _close(run([3, L - 3], with_bias=False), nb, tol, "no bias")


@pytest.mark.parametrize("dtype", [F32, B16])
def test_xielu_both_sides_and_pad_columns(dtype):
    M, Fw, ldz, ldo = 7, 77, 96, 128
    g = torch.Generator().manual_seed(3)
    z = _bf(torch.randn(M, ldz, generator=g) * 3)
    z[0, :4] = torch.tensor([0.0, -0.0, 20.0, -30.0]).to(B16)
    lib = _lib.lib()
    for pq in ([0.3, 0.8], [-4.0, 6.0], [30.0, -30.0]):
        coef = _bf(torch.tensor(pq))
        zd, out = z.to(DEV, dtype), torch.full((M, ldo), 7.0, dtype=dtype, device=DEV)
        cd = coef.to(DEV)
        check(lib.evo_xielu(ptr(zd), ldz, ptr(cd), ptr(out), ldo, M, Fw, 1 if dtype == F32 else 0, _stream()))
        want = O.xielu(z[:, :Fw].double(), coef[0].double(), coef[1].double())
        _close(out[:, :Fw], want, 1e-6 if dtype == F32 else 6e-3, f"xielu {pq}")
        assert (out[:, Fw:] == 0).all()


@pytest.mark.parametrize("width,groups", [(24, 3), (128, 2), (130, 1), (96, 96), (1040, 8)])
@pytest.mark.parametrize("dtype", [F32, B16])
def test_gated_group_norm(width, groups, dtype):
    M, eps, ldg = 5, 1e-5, width + 16
    ldo = (width + 63) // 64 * 64
    g = torch.Generator().manual_seed(width)
    y, gate, nw = torch.randn(M, width, generator=g), _bf(torch.randn(M, ldg, generator=g)), _bf(1 + 0.3 * torch.randn(width, generator=g))
    gated = y.double() * O.silu(gate[:, :width].double())
    want = O.rms(gated.view(M, groups, width // groups), eps).reshape(M, width) * nw.double()
    out = torch.full((M, ldo), 7.0, dtype=dtype, device=DEV)
    yd, gd, nwd = y.to(DEV), gate.to(DEV, dtype), nw.to(DEV)
    check(_lib.lib().evo_gated_group_norm(ptr(yd), ptr(gd), ldg, ptr(nwd), ptr(out), ldo, M, width, groups, eps, 1 if dtype == F32 else 0, _stream()))
    _close(out[:, :width], want, 1e-6 if dtype == F32 else 6e-3, "gated group norm")
    assert (out[:, width:] == 0).all()


# ------------------------------------------------------------------ mixers alone (one layer, no feed-forward)
def _one_side(W, side):
    """A parallel layer whose other mixer contributes nothing: its closing norm weight is zero."""
    W = dict(W)
    other = "right" if side == "left" else "left"
    W[f"l0.mix.{other}.out"] = torch.zeros_like(W[f"l0.mix.{other}.out"])
    return W


DELTA_SIZES = [dict(heads=2, kv_heads=1, dim=8, vdim=12, taps=3), dict(heads=3, kv_heads=3, dim=20, vdim=5, taps=4), dict(heads=4, kv_heads=2, dim=64, vdim=64, taps=2),
               dict(heads=1, kv_heads=1, dim=3, vdim=40, taps=1), dict(heads=2, kv_heads=1, dim=136, vdim=24, taps=4), dict(heads=6, kv_heads=2, dim=32, vdim=130, taps=4)]


@pytest.mark.parametrize("sizes", DELTA_SIZES, ids=lambda s: "h{heads}g{kv_heads}k{dim}v{vdim}t{taps}".format(**s))
def test_gated_delta_mixer_matches_the_oracle(sizes):
    cfg = O.make_config(layers=("delta",), no_ff_layers=(0,), width=40, **sizes)
    W = O.random_weights(cfg, seed=sizes["dim"])
    tokens = _tokens(cfg, 45)
    want = O.forward(cfg, W, tokens)
    model = _model(cfg, W)
    got, _ = model(torch.tensor([tokens], device=DEV))
    _close(got[0], want, 2e-5, "whole")
    _close(_portions(model, tokens, [1] * 45), want, 2e-5, "steps")
    _close(_portions(model, tokens, [17, 2, 1, 16, 2, 7]), want, 2e-5, "portions across the staging rounds")


SSD_SIZES = [dict(ssd_heads=4, ssd_vdim=6, state=5, groups=2, norm_groups=3, ssd_taps=2), dict(ssd_heads=2, ssd_vdim=64, state=16, groups=1, norm_groups=1, ssd_taps=4),
             dict(ssd_heads=3, ssd_vdim=10, state=130, groups=3, norm_groups=5, ssd_taps=3), dict(ssd_heads=8, ssd_vdim=33, state=48, groups=2, norm_groups=8, ssd_taps=1)]


@pytest.mark.parametrize("sizes", SSD_SIZES, ids=lambda s: "h{ssd_heads}v{ssd_vdim}n{state}g{groups}".format(**s))
def test_state_space_mixer_matches_the_oracle(sizes):
    cfg = O.make_config(layers=("parallel",), no_ff_layers=(0,), width=40, **sizes)
    W = _one_side(O.random_weights(cfg, seed=sizes["state"]), "right")
    tokens = _tokens(cfg, 45)
    want = O.forward(cfg, W, tokens)
    model = _model(cfg, W)
    got, _ = model(torch.tensor([tokens], device=DEV))
    _close(got[0], want, 2e-5, "whole")
    _close(_portions(model, tokens, [1] * 45), want, 2e-5, "steps")
    _close(_portions(model, tokens, [17, 2, 1, 16, 2, 7]), want, 2e-5, "portions")


def test_state_space_mixer_with_sixteen_lanes_per_column_on_a_long_prompt():
    """Prompts of 256 tokens or more on few heads of 65 to 128 state rows put 16 lanes on a state column; shorter portions continue with 8."""
    cfg = O.make_config(layers=("parallel",), no_ff_layers=(0,), width=40, ssd_heads=2, ssd_vdim=40, state=128, groups=1, norm_groups=2, ssd_taps=2)
    W = _one_side(O.random_weights(cfg, seed=17), "right")
    tokens = _tokens(cfg, 300)
    want = O.forward(cfg, W, tokens)
    model = _model(cfg, W)
    got, _ = model(torch.tensor([tokens], device=DEV))
    _close(got[0], want, 2e-5, "whole")
    _close(_portions(model, tokens, [12, 260, 1, 27]), want, 2e-5, "a long portion on a carried state, a step, a portion")


ATT_SIZES = [dict(att_heads=4, att_kv_heads=2, att_dim=12, att_vdim=10, window=9, pool=3, rot_dims=8), dict(att_heads=3, att_kv_heads=3, att_dim=16, att_vdim=16, window=7, pool=4, rot_dims=16),
             dict(att_heads=2, att_kv_heads=1, att_dim=40, att_vdim=136, window=33, pool=1, rot_dims=0), dict(att_heads=5, att_kv_heads=1, att_dim=6, att_vdim=3, window=1, pool=2, rot_dims=2),
             dict(att_heads=2, att_kv_heads=2, att_dim=8, att_vdim=8, window=200, pool=5, rot_dims=4), dict(att_heads=2, att_kv_heads=2, att_dim=24, att_vdim=8, window=12, pool=0, rot_dims=6, softcap=0.0)]


@pytest.mark.parametrize("sizes", ATT_SIZES, ids=lambda s: "h{att_heads}g{att_kv_heads}k{att_dim}v{att_vdim}w{window}p{pool}r{rot_dims}".format(**s))
def test_pooled_window_attention_mixer_matches_the_oracle(sizes):
    cfg = O.make_config(layers=("parallel",), no_ff_layers=(0,), width=40, **sizes)
    W = _one_side(O.random_weights(cfg, seed=sizes["window"]), "left")
    tokens = _tokens(cfg, 70)
    want = O.forward(cfg, W, tokens)
    model = _model(cfg, W)
    got, _ = model(torch.tensor([tokens], device=DEV))
    _close(got[0], want, 2e-5, "whole")
    _close(_portions(model, tokens, [1] * 70), want, 2e-5, "steps")
    _close(_portions(model, tokens, [17, 2, 1, 16, 2, 7, 3, 22]), want, 2e-5, "portions")
    bf = _model(cfg, W, B16)
    rel = lambda a, b: ((a.double().cpu() - b.double().cpu()).pow(2).mean().sqrt() / b.double().pow(2).mean().sqrt()).item()
    whole16, _ = bf(torch.tensor([tokens], device=DEV))
    assert rel(whole16[0], want) < 3e-2 and rel(_portions(bf, tokens, [30] + [1] * 40), want) < 3e-2


@pytest.mark.parametrize("H,G,dk,dv,window,pool,cap,L", [(4, 2, 64, 64, 70, 8, 20.0, 300), (2, 2, 128, 128, 130, 64, 0.0, 400), (3, 1, 32, 24, 16, 1, 5.0, 150),
                                                        (2, 1, 16, 8, 200, 3, 50.0, 330)])
def test_attention_kernels_agree_on_tokens_blocks_sink_and_cap(H, G, dk, dv, window, pool, cap, L):
    """The three kernels behind evo_window_attn_fwd on the same bf16 cache: the tensor-core kernel (all rows in one call), the
    many-query CUDA-core kernel (fp32 copies of the same numbers) and the few-query kernel (one row per call), against a plain
    softmax over the visible tokens and pooled rows with the sink in the denominator."""
    from evo_b200._lib import WindowAttnParams
    g = torch.Generator().manual_seed(L)
    scale = 2.5 / math.sqrt(dk)                            # scores of a few units either way, so that the cap bends them
    q = _bf(torch.randn(L, H * dk, generator=g))
    kv = _bf(torch.randn(L + 5, G * (dk + dv), generator=g))
    sink = _bf(torch.randn(H, generator=g) * 2)
    lib = _lib.lib()
    ldo = (H * dv + 63) // 64 * 64
    nb = L // pool + 1

    def run(dtype, rows_per_call):
        dt = 1 if dtype == F32 else 0
        qd, kvd, sd = q.to(DEV, dtype), kv.to(DEV, dtype).contiguous(), sink.to(DEV)
        pooled = torch.full((nb, G * (dk + dv)), float("nan"), dtype=dtype, device=DEV)
        row = G * (dk + dv)
        check(lib.evo_pool_rows(ptr(kvd), row, kvd.numel(), ptr(pooled), row, pooled.numel(), 1, L, row, pool, 0, None, dt, _stream()))
        out = torch.empty(L, ldo, dtype=dtype, device=DEV)
        esz = qd.element_size()
        for r0 in range(0, L, rows_per_call):
            n = min(rows_per_call, L - r0)
            ap = WindowAttnParams(q=qd.data_ptr() + r0 * H * dk * esz, q_tok_stride=H * dk, k=kvd.data_ptr(), v=kvd.data_ptr() + G * dk * esz, k_tok_stride=row, v_tok_stride=row,
                                  k_batch_stride=kvd.numel(), v_batch_stride=kvd.numel(), out=out.data_ptr() + r0 * ldo * esz, ldo=ldo, dtype=dt, B=1, Lq=n, H=H, G=G,
                                  dk=dk, dv=dv, n_maps=1, q_pos0=r0, window=window, scale=scale, softcap=cap, sink=sd.data_ptr(), pool=pool,
                                  pool_k=pooled.data_ptr(), pool_v=pooled.data_ptr() + G * dk * esz, pool_tok_stride=row, pool_batch_stride=pooled.numel())
            check(lib.evo_window_attn_fwd(C.byref(ap), _stream()))
        return out[:, :H * dv].double().cpu(), pooled

    qf, kf = q.double().view(L, H, dk), kv.double()
    want = torch.zeros(L, H, dv, dtype=torch.float64)
    pk = torch.stack([kf[b * pool:(b + 1) * pool].mean(0) for b in range(L // pool)]) if L >= pool else kf[:0]
    for h in range(H):
        gi = h // (H // G)
        for i in range(L):
            js, bs = O.visible_tokens(i, window), O.visible_blocks(i, window, pool)
            rows = torch.cat([kf[js], pk[bs]]) if bs else kf[js]
            sc = rows[:, gi * dk:(gi + 1) * dk] @ qf[i, h] * scale
            if cap > 0:
                sc = cap * torch.tanh(sc / cap)
            mx = torch.maximum(sc.max(), sink[h].double())
            e = torch.exp(sc - mx)
            want[i, h] = (e[:, None] * rows[:, G * dk + gi * dv:G * dk + (gi + 1) * dv]).sum(0) / (e.sum() + torch.exp(sink[h].double() - mx))
    want = want.view(L, H * dv)
    many32, pooled32 = run(F32, L)
    _close(pooled32[:L // pool, :], pk, 1e-6, "pooled rows")
    _close(many32, want, 2e-5, "many-query kernel, fp32")
    _close(run(F32, 1)[0], want, 2e-5, "few-query kernel, fp32")
    _close(run(F32, 3)[0], want, 2e-5, "few-query kernel, three rows a call")
    # bf16: pooled rows are rounded when stored, outputs when written
    tensor, _ = run(B16, L)
    few, _ = run(B16, 2)
    _close(tensor, want, 1.5e-2, "tensor-core kernel")
    _close(few, want, 1.5e-2, "few-query kernel, bf16")
    _close(tensor, few, 1e-2, "tensor-core kernel against the few-query kernel")


# ------------------------------------------------------------------ edges of the window and of the pooled blocks
def _dominant_token(cfg, W, plain, odd, gain):
    """Weights under which the key of token `odd` beats the key of token `plain` by `gain` in every head, for a query of `plain`, at
    any distance: no rotation and no soft cap in the configuration, the other mixer silenced, the sink far below every score, and the
    per-entry query norm weights scaled head by head."""
    a = cfg["layers"][0]["mixer"]["left"]
    H, G, dk = a["heads"], a["kv_heads"], a["dim"]
    eps = cfg["norm"]["eps"]
    w = {k: v.double() for k, v in W.items()}
    h = O.rms(w["embed"][[plain, odd]], eps) * w["l0.norm1"]
    q = (O.rms(h @ w["l0.mix.left.q"].T + w["l0.mix.left.q.b"], eps) * w["l0.mix.left.q.norm"]).view(2, H, dk)
    k = (O.rms(h @ w["l0.mix.left.k"].T + w["l0.mix.left.k.b"], eps) * w["l0.mix.left.k.norm"]).view(2, G, dk)
    out = _one_side(W, "left")
    qn = W["l0.mix.left.q.norm"].double().view(H, dk).clone()
    for hd in range(H):
        g = hd // (H // G)
        delta = float(q[0, hd] @ (k[1, g] - k[0, g])) * a["scale"]
        qn[hd] *= gain / delta
    out["l0.mix.left.q.norm"] = qn.view(-1).to(B16)
    out["l0.mix.left.sink"] = torch.full_like(W["l0.mix.left.sink"], -1000.0)      # the scaled scores may all be far below zero: keep the sink below them
    return out


_EDGE_ORACLE = {}


def _edge_case(window, pool, T_extra=6):
    """(config, weights, plain prompt, prompt with the other token at j, oracle logits of both) -- shared by the dtypes."""
    key = (window, pool)
    if key not in _EDGE_ORACLE:
        cfg = O.make_config(layers=("parallel",), no_ff_layers=(0,), window=window, pool=pool, rot_dims=0, softcap=0.0, att_heads=2, att_kv_heads=1, att_dim=16, att_vdim=16,
                            width=64, vocab=50)
        W = _dominant_token(cfg, O.random_weights(cfg, seed=window), 7, 31, 10.0 * pool)
        j = pool + 1                                          # second entry of block 1
        T = (j // pool) * pool + pool - 1 + window + T_extra
        plain, odd = [7] * T, [7] * T
        odd[j] = 31
        _EDGE_ORACLE[key] = (cfg, W, plain, odd, j, O.forward(cfg, W, plain), O.forward(cfg, W, odd))
    return _EDGE_ORACLE[key]


@pytest.mark.parametrize("dtype", [F32, B16])
@pytest.mark.parametrize("window,pool", [(5, 3), (40, 8), (3, 5), (96, 7)])
def test_window_and_block_edges_with_one_dominant_token(dtype, window, pool):
    """Equal tokens with one other token at position j whose key dominates every softmax that sees it.  Position j + window - 1 is the
    last that sees the token itself; then nobody sees it until its block has wholly left the window, at position e = b*pool + pool - 1
    + window, from where its pooled key (boosted so that the block's mean dominates too) is seen for good.  The stream rows differ only
    at j, so in between the logits equal the plain prompt's -- in a prompt, in portions cut at the edges, and in single steps."""
    cfg, W, plain, odd, j, want_plain, want_odd = _edge_case(window, pool)
    model = _model(cfg, W, dtype)
    T = len(odd)
    seen_again = (j // pool) * pool + pool - 1 + window
    last_in = j + window - 1
    scale = want_plain.abs().max().item()
    tol_same = 1e-5 if dtype == F32 else 2e-2
    d_want = (want_odd - want_plain).abs().max(-1).values / scale
    assert d_want[last_in] > 0.1 and d_want[seen_again:].min() > 3 * 2e-2, "the case does not show the edges"
    if seen_again > last_in + 1:
        assert d_want[last_in + 1:seen_again].max() < 1e-9
    base, _ = model(torch.tensor([plain], device=DEV))
    cuts = sorted({j + 1, last_in, last_in + 1, seen_again, seen_again + 1, T} - {0})
    sizes = [b - a for a, b in zip([0] + cuts[:-1], cuts) if b > a]
    for name, parts in (("prompt", [T]), ("portions", sizes), ("steps", [j + 1] + [1] * (T - j - 1)), ("two by two", [2] * (T // 2) + [1] * (T % 2))):
        got = _portions(model, odd, parts)
        d = (got - base[0]).abs().max(-1).values.double().cpu() / scale
        assert d[last_in] > 0.5 * d_want[last_in], f"{name}: the token at the window's inner edge is not seen ({d[last_in]:.2e})"
        if seen_again > last_in + 1:
            assert d[last_in + 1:seen_again].max() < tol_same, f"{name}: a token outside the window is seen before its block is ({d[last_in + 1:seen_again].max():.2e})"
        assert (d[seen_again:] > 0.5 * d_want[seen_again:]).all(), f"{name}: the block is not seen from its first position on"
        if dtype == F32:
            _close(got, want_odd, 2e-5, name)


@pytest.mark.parametrize("dtype", [F32, B16])
def test_far_key_among_hundreds_is_kept_through_its_block(dtype):
    cfg = O.make_config(layers=("parallel",), no_ff_layers=(0,), window=64, pool=8, rot_dims=0, softcap=0.0, att_heads=2, att_kv_heads=2, att_dim=16, att_vdim=16, width=64, vocab=50)
    W = _dominant_token(cfg, O.random_weights(cfg, seed=5), 7, 31, 80.0)
    model = _model(cfg, W, dtype)
    T, j = 700, 3
    plain, odd = [7] * T, [7] * T
    odd[j] = 31
    base, _ = model(torch.tensor([plain], device=DEV))
    scale = base.abs().max().item()
    for name, parts in (("prompt", [T]), ("prompt then steps", [600] + [1] * 100), ("portions", [250, 250, 2, 198])):
        got = _portions(model, odd, parts)
        d = (got - base[0]).abs().max(-1).values / scale
        assert d[7 + 64:].min() > 0.04, f"{name}: the far block is lost ({d[7 + 64:].min():.2e})"
        assert d[j + 64:7 + 64].max() < (1e-5 if dtype == F32 else 2e-2), name
    if dtype == F32:
        rows = [0, j, j + 63, j + 64, 70, 71, 72, 300, 699]
        m = cfg["layers"][0]["mixer"]["left"]
        # the oracle's attention on the wanted rows only (the layer is attention alone: the other mixer's closing weight is zero)
        w = {k: v.double() for k, v in W.items()}
        eps = cfg["norm"]["eps"]
        x = w["embed"][torch.tensor(odd)]
        left = {k[len("l0.mix.left."):]: t for k, t in w.items() if k.startswith("l0.mix.left.")}
        a = O.pooled_window_attention(O.rms(x, eps) * w["l0.norm1"], left, m, eps, rows=rows)
        xr = (x + 0.5 * O.rms(a, eps) * w["l0.mix.left.out"])[rows]
        want = (O.rms(xr, eps) * w["final.norm"]) @ w["head"].T
        _close(got[rows], want, 2e-5, "far rows against the oracle")


# ------------------------------------------------------------------ the model
CONFIGS = {
    "mixed": dict(),
    "delta_first": dict(layers=("delta_2", "parallel", "delta", "parallel"), no_ff_layers=(1,), width=72, vocab=257, window=4, pool=4, rot_dims=12, norm_groups=1, groups=1,
                        kv_heads=2, att_kv_heads=4),
    "no_ff_no_pool": dict(layers=("parallel", "delta"), no_ff_layers=(0, 1), pool=0, rot_dims=0, softcap=0.0, taps=1, ssd_taps=1, heads=1, kv_heads=1, att_heads=1, att_kv_heads=1,
                          ssd_heads=1, groups=1, norm_groups=1),
    "odd": dict(layers=("delta", "parallel", "delta_2"), width=50, ff=37, vocab=33, heads=3, kv_heads=1, dim=5, vdim=7, taps=2, att_heads=3, att_kv_heads=1, att_dim=10, att_vdim=9,
                window=7, pool=2, rot_dims=6, ssd_heads=3, ssd_vdim=5, state=7, groups=1, norm_groups=3, ssd_taps=3),
    "wide": dict(layers=("parallel", "delta"), width=200, ff=264, heads=2, kv_heads=2, dim=72, vdim=136, taps=4, att_heads=2, att_kv_heads=1, att_dim=72, att_vdim=40, window=1000, pool=16,
                 rot_dims=72, ssd_heads=2, ssd_vdim=136, state=70, groups=2, norm_groups=2, ssd_taps=4),
}


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_model_whole_steps_and_portions_match_the_oracle_in_fp32(name):
    cfg = O.make_config(**CONFIGS[name])
    W = O.random_weights(cfg, seed=len(name))
    T = 75
    tokens = _tokens(cfg, T)
    streams = []
    want = O.forward(cfg, W, tokens, taps=streams)
    model = _model(cfg, W)
    model._tap = []
    got, _ = model(torch.tensor([tokens], device=DEV))
    assert len(model._tap) == len(streams)
    for r, (a, b) in enumerate(zip(model._tap, streams)):
        _close(a, b, 2e-5, f"{name}: residual stream after layer {r}")
    model._tap = None
    _close(got[0], want, 2e-5, f"{name}: whole")
    _close(_portions(model, tokens, [1] * T), want, 2e-5, f"{name}: token by token from the first token")
    _close(_portions(model, tokens, [40] + [1] * 35), want, 2e-5, f"{name}: prompt then steps")
    _close(_portions(model, tokens, [2, 2, 3, 30, 1, 2, 17, 9, 2, 5, 2]), want, 2e-5, f"{name}: portions")
    _close(_portions(model, tokens[:1], [1]), want[:1], 2e-5, f"{name}: a one-token sequence")
    _close(_portions(model, tokens[:2], [2]), want[:2], 2e-5, f"{name}: a two-token sequence")


def test_layers_with_their_own_sizes_and_a_cache_that_has_to_grow():
    cfg = O.make_config(layers=("parallel", "delta", "parallel", "delta_3"), width=104, vocab=211)
    cfg["layers"][2]["mixer"]["left"] = {"heads": 6, "kv_heads": 3, "dim": 8, "vdim": 40, "scale": 0.2, "mask": {"size": 3, "pool": 2}, "rot": {"base": 7.0, "dims": 6}, "softcap": 2.0}
    cfg["layers"][2]["mixer"]["right"] = {"heads": 2, "vdim": 24, "state": 9, "groups": 1, "norm_groups": 4, "conv": 5}
    cfg["layers"][3]["mixer"] = {"heads": 4, "kv_heads": 4, "dim": 16, "vdim": 8, "conv": 2}
    cfg["layers"][1]["mlp"] = None
    cfg["layers"][3]["mlp"]["ff"] = 72
    W = O.random_weights(cfg, seed=21)
    tokens = _tokens(cfg, 70, seed=8)
    want = O.forward(cfg, W, tokens)
    model = _model(cfg, W)
    got, _ = model(torch.tensor([tokens], device=DEV))
    _close(got[0], want, 2e-5, "whole")
    state = model.initialize_inference_params(max_seqlen=16, max_batch_size=1)
    _close(_portions(model, tokens, [9, 2, 20, 1, 1, 30, 7], state=state), want, 2e-5, "portions through a growing cache")
    assert all(model._cache_tokens(k, c) >= 70 for k, c in state["mha"].key_value_memory_dict.items())


def test_model_bf16_stays_within_rounding_of_the_oracle_and_of_itself():
    cfg = O.make_config()
    W = O.random_weights(cfg, seed=3)
    tokens = _tokens(cfg, 90, seed=2)
    want = O.forward(cfg, W, tokens)
    model = _model(cfg, W, B16)
    whole, _ = model(torch.tensor([tokens], device=DEV))
    cut = _portions(model, tokens, [50, 2, 1, 1, 30, 6])
    rel = lambda a, b: ((a.double().cpu() - b.double().cpu()).pow(2).mean().sqrt() / b.double().pow(2).mean().sqrt()).item()
    assert rel(whole[0], want) < 3e-2
    assert rel(cut, want) < 3e-2
    assert rel(cut, whole[0].cpu()) < 3e-2
    model.gemm_path = "simt"                              # the tensor-core linear layers against the CUDA-core ones
    simt, _ = model(torch.tensor([tokens], device=DEV))
    assert rel(simt[0], whole[0].cpu()) < 2e-2


def test_batch_rows_equal_each_sequence_alone_and_wanted_rows_select():
    cfg = O.make_config()
    W = O.random_weights(cfg, seed=5)
    model = _model(cfg, W)
    ids = torch.randint(0, cfg["vocab"], (3, 33), generator=torch.Generator().manual_seed(4)).to(DEV)
    both, _ = model(ids)
    for b in range(3):
        alone, _ = model(ids[b:b + 1])
        _close(both[b], alone[0].double().cpu(), 1e-6, f"row {b}")
    state = model.initialize_inference_params(max_seqlen=64, max_batch_size=3)
    a, _ = model(ids[:, :20], inference_params_dict=state)
    state["mha"].seqlen_offset = state["hyena"].seqlen_offset = 20
    b_, _ = model(ids[:, 20:], inference_params_dict=state)
    _close(torch.cat([a, b_], 1), both.double().cpu(), 1e-5, "batched portions")
    rows = [0, 7, 32, 40, 98]
    picked, _ = model(ids, logits_rows=rows)
    _close(picked, both.reshape(-1, both.shape[-1])[rows].double().cpu(), 1e-6, "wanted rows")


def test_reused_state_memory_and_long_decoding_past_the_window():
    """State holders that still hold another request's rows, pooled rows, matrix states and carried inputs (and NaNs beyond) serve a
    new request; decoding runs far past the window; a request interleaved with another one keeps its own state."""
    cfg = O.make_config(window=11, pool=4)
    W = O.random_weights(cfg, seed=7)
    model = _model(cfg, W)
    a, b = _tokens(cfg, 120, seed=6), _tokens(cfg, 60, seed=9)
    want_a, want_b = O.forward(cfg, W, a), O.forward(cfg, W, b)
    state = model.initialize_inference_params(max_seqlen=128, max_batch_size=1)
    _close(_portions(model, a, [20] + [1] * 100, state=state), want_a, 2e-5, "long decoding")
    for key, cache in state["mha"].key_value_memory_dict.items():
        cache[:, (100 if key >= 0 else 25):, :3] = float("nan")
    _close(_portions(model, b, [7, 2, 51], state=state), want_b, 2e-5, "the same holders, used again from position 0")
    sa = model.initialize_inference_params(max_seqlen=128, max_batch_size=1)
    sb = model.initialize_inference_params(max_seqlen=128, max_batch_size=1)
    outs_a, outs_b = [], []
    for lo, hi in ((0, 30), (30, 31), (31, 60)):
        for tokens, st, outs in ((a, sa, outs_a), (b, sb, outs_b)):
            st["mha"].seqlen_offset = st["hyena"].seqlen_offset = lo
            lg, _ = model(torch.tensor([tokens[lo:hi]], device=DEV), inference_params_dict=st)
            outs.append(lg[0])
    _close(torch.cat(outs_a), want_a[:60], 2e-5, "interleaved a")
    _close(torch.cat(outs_b), want_b[:60], 2e-5, "interleaved b")


@pytest.mark.parametrize("device_loop", [True, False])
def test_greedy_generation_through_the_generator(device_loop):
    from evo_b200 import CharLevelTokenizer, Generator
    cfg = O.make_config(vocab=512)
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
    cfg = O.make_config(vocab=512)
    W = O.random_weights(cfg, seed=13)
    ckpt = str(tmp_path / "ckpt")
    _write_checkpoint(ckpt, cfg, W)
    texts, scores = cli.main(["--model-dir", ckpt, "--prompt", "ACGTTGCA", "--n-samples", "2", "--n-tokens", "9", "--top-k", "1", "--device", DEV, "--verbose", "0"])
    assert len(texts) == 2 and texts[0] == texts[1] and len(scores) == 2
    tokens = _tokens(cfg, 40, seed=5)
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
