"""Gakupel on the GPU against the plain oracle (oracle/gakupel_oracle.py): the new row kernels alone, the router, every mixer alone
over several sizes, the attention kernels against one another, then the model -- whole prompts, token-by-token decoding, portions down
to two tokens, batches, reused state memory, far keys, the steps of the query temperature, the first tokens of a sequence, long
decoding, other sizes -- and greedy generation through the framework's Generator and command line.  Small configurations, random
weights; where random weights would hide a fault the weights are made so that it shows."""
import ctypes as C
import math

import pytest
import torch

from evo_b200 import _lib
from evo_b200._lib import MoeRouteParams, PostNormParams, QkPrepParams, WindowAttnParams, check, ptr
from oracle import gakupel_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F32, B16, F64 = torch.float32, torch.bfloat16, torch.float64


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _bf(t):
    return t.to(B16)


def _close(got, want, tol, what=""):
    err = (got.double().cpu() - want.double().cpu()).abs().max().item()
    ref = max(want.abs().max().item(), 1e-6)
    assert err <= tol * ref, f"{what}: max err {err:.3e} vs scale {ref:.3e} (tol {tol})"


def _model(cfg, W, dtype=F32):
    from evo_b200.gakupel import Gakupel, GakupelConfig
    m = Gakupel(GakupelConfig.from_dict(cfg), dtype=dtype)
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
def test_post_norm_sums_norms_files_mixes_and_gathers(D, ldo, dtype):
    M, eps, slots = 6, 1e-5, 4
    g = torch.Generator().manual_seed(D)
    x = torch.randn(M, D, generator=g)
    ys = [_bf(torch.randn(M, D + 8 * b, generator=g) * 3 + 1.5) for b in range(2)]        # a mean far from zero: the variance is about the mean
    scales = [1.25, 0.5]
    nw, nb, fw, fb = (_bf(torch.randn(D, generator=g)) for _ in range(4))
    mw = _bf(torch.randn(slots, generator=g))
    stack = torch.randn(slots, M, D, generator=g)
    t = sum(s * y[:, :D].double() for s, y in zip(scales, ys))
    x1 = x.double() + O.layer_norm(t, nw.double(), nb.double(), eps)
    mixed = sum(mw[j].double() * stack[j].double() for j in range(slots - 1)) + mw[slots - 1].double() * x1
    dt = 1 if dtype == F32 else 0
    tol = 2e-6 if dtype == F32 else 6e-3
    yd = [y.to(DEV, dtype) for y in ys]
    nwd, nbd, fwd, fbd, mwd = (v.to(DEV) for v in (nw, nb, fw, fb, mw))
    lib = _lib.lib()

    def params(xd, n_in, out=None, rows=M, mix=None, out_norm=False, gather=None, x_in=None):
        p = PostNormParams(x=xd.data_ptr(), x_in=x_in.data_ptr() if x_in is not None else None, n_in=n_in, eps=eps, dtype=dt, rows=rows, D=D,
                           out=out.data_ptr() if out is not None else None, ldo=ldo, gather=gather.data_ptr() if gather is not None else None)
        for b in range(n_in):
            p.y[b], p.ldy[b], p.scale[b] = yd[b].data_ptr(), D + 8 * b, scales[b]
        if n_in:
            p.norm_w, p.norm_b = nwd.data_ptr(), nbd.data_ptr()
        if mix is not None:
            p.stack, p.stack_stride, p.mix_n, p.mix_w = mix.data_ptr(), mix.stride(0), slots, mwd.data_ptr()
        if out_norm:
            p.out_norm_w, p.out_norm_b = fwd.data_ptr(), fbd.data_ptr()
        return p
    # two inputs, norm, plain copy out
    xd, o = x.to(DEV), torch.full((M, ldo), 7.0, dtype=dtype, device=DEV)
    check(lib.evo_post_norm(C.byref(params(xd, 2, o)), _stream()))
    _close(xd, x1, 2e-6, "stream")
    _close(o[:, :D], x1, tol, "copy of the stream")
    assert (o[:, D:] == 0).all()
    # the same with the result filed in the last slot and the mix handed on
    xd, sd, o = x.to(DEV), stack.to(DEV), torch.full((M, ldo), 7.0, dtype=dtype, device=DEV)
    check(lib.evo_post_norm(C.byref(params(xd, 2, o, mix=sd)), _stream()))
    _close(sd[slots - 1], x1, 2e-6, "filed result")
    assert torch.equal(sd[:slots - 1].cpu(), stack[:slots - 1])
    _close(xd, mixed, 4e-6, "mixed stream")
    _close(o[:, :D], mixed, tol, "copy of the mixed stream")
    # gathered rows with the closing norm: nothing but the output is written
    xd, sd, o = x.to(DEV), stack.to(DEV), torch.full((2, ldo), 7.0, dtype=dtype, device=DEV)
    rows = torch.tensor([4, 1], device=DEV)
    check(lib.evo_post_norm(C.byref(params(xd, 2, o, rows=2, mix=sd, out_norm=True, gather=rows)), _stream()))
    _close(o[:, :D], O.layer_norm(mixed, fw.double(), fb.double(), eps)[[4, 1]], 4e-6 if dtype == F32 else 1e-2, "closing norm of gathered rows")
    assert torch.equal(xd.cpu(), x) and torch.equal(sd.cpu(), stack) and (o[:, D:] == 0).all()
    # no input: copy from another buffer; one input
    xd, src, o = torch.zeros(M, D, device=DEV), x.to(DEV), torch.full((M, ldo), 7.0, dtype=dtype, device=DEV)
    check(lib.evo_post_norm(C.byref(params(xd, 0, o, x_in=src)), _stream()))
    assert torch.equal(xd.cpu(), x)
    _close(o[:, :D], x, tol, "copy")
    xd = x.to(DEV)
    check(lib.evo_post_norm(C.byref(params(xd, 1)), _stream()))
    _close(xd, x.double() + O.layer_norm(scales[0] * ys[0][:, :D].double(), nw.double(), nb.double(), eps), 2e-6, "one input, no output")


@pytest.mark.parametrize("H,G,dk,dv,rot,per_head,every", [(4, 2, 16, 16, 8, True, 0), (3, 1, 10, 9, 6, False, 4), (2, 2, 64, 40, 0, False, 192), (6, 2, 64, 64, 16, True, 0),
                                                          (1, 1, 7, 5, 2, True, 1)])
@pytest.mark.parametrize("dtype", [F32, B16])
def test_qk_prep_head_norms_rotation_and_temperature(H, G, dk, dv, rot, per_head, every, dtype):
    L, pos0, eps, coef = 9, 250, 1e-5, 0.35
    g = torch.Generator().manual_seed(H * dk + rot)
    qw, kw, vw = H * dk, G * dk, G * dv
    ld = qw + kw + vw + 3
    z = _bf(torch.randn(L, ld, generator=g))
    qn = _bf(1 + 0.3 * torch.randn(dk if per_head else qw, generator=g))
    kn = _bf(1 + 0.3 * torch.randn(dk if per_head else kw, generator=g))
    pos = torch.arange(pos0, pos0 + L)
    q, k, v = z[:, :qw].double(), z[:, qw:qw + kw].double(), z[:, qw + kw:qw + kw + vw].double()
    if per_head:
        qr = (O.rms(q.view(L, H, dk), eps) * qn.double()).view(L, H, dk)
        kr = (O.rms(k.view(L, G, dk), eps) * kn.double()).view(L, G, dk)
    else:
        qr, kr = (O.rms(q, eps) * qn.double()).view(L, H, dk), (O.rms(k, eps) * kn.double()).view(L, G, dk)
    qr, kr = O.rotate_half(qr, pos, rot, 500.0), O.rotate_half(kr, pos, rot, 500.0)
    if every:
        qr = qr * (1 + coef * torch.log(torch.div(pos + 1, every, rounding_mode="floor").double() + 1))[:, None, None]
    freq = (500.0 ** (-2.0 * torch.arange(rot // 2, dtype=F64) / max(rot, 1))).to(F32).to(DEV)
    zd = z.to(DEV, dtype)
    cache = torch.zeros(1, pos0 + L + 2, kw + vw, dtype=dtype, device=DEV)
    esz = zd.element_size()
    qn_d, kn_d = qn.to(DEV), kn.to(DEV)
    p = QkPrepParams(q=zd.data_ptr(), k=zd.data_ptr() + qw * esz, v=zd.data_ptr() + (qw + kw) * esz, ld=ld, q_norm_w=qn_d.data_ptr(), k_norm_w=kn_d.data_ptr(),
                     eps=eps, freq=freq.data_ptr() if rot else None, rot_dims=rot, cache=cache.data_ptr(), cache_row=kw + vw, cache_batch_stride=cache.shape[1] * (kw + vw),
                     B=1, L=L, H=H, G=G, dk=dk, dv=dv, pos0=pos0, dtype=1 if dtype == F32 else 0, norm_per_head=int(per_head), q_temp_coef=coef, q_temp_every=every)
    check(_lib.lib().evo_qk_prep(C.byref(p), _stream()))
    tol = 3e-5 if dtype == F32 else 8e-3
    _close(zd[:, :qw], qr.reshape(L, qw), tol, "queries")
    _close(cache[0, pos0:pos0 + L, :kw], kr.reshape(L, kw), tol, "keys in the cache")
    _close(cache[0, pos0:pos0 + L, kw:], v, 1e-6 if dtype == F32 else 8e-3, "values in the cache")
    assert (cache[0, :pos0] == 0).all() and (cache[0, pos0 + L:] == 0).all()


@pytest.mark.parametrize("E,top,groups,keep,extra,M", [(8, 3, 4, 2, 1, 37), (12, 3, 4, 2, 1, 1100), (6, 3, 3, 2, 0, 5), (16, 4, 0, 0, 1, 9), (64, 6, 8, 3, 1, 40), (5, 5, 5, 5, 0, 3),
                                                       (4, 1, 4, 1, 1, 2)])
@pytest.mark.parametrize("dtype", [F32, B16])
def test_router_scores_groups_choice_and_weights(E, top, groups, keep, extra, M, dtype):
    D = 50 if E == 6 else 64
    g = torch.Generator().manual_seed(E + M)
    h = _bf(torch.randn(M, D, generator=g))
    rw = _bf(torch.randn(E + extra, D, generator=g) / 3)
    corr = _bf(torch.randn(E, generator=g) * 0.4)
    r = {"experts": E, "top": top, "scale": 1.7}
    if groups:
        r["groups"] = {"count": groups, "keep": keep}
    want = O.route(h.double(), {"router": rw[:E].double(), "correction": corr.double()}, r)
    hd, rwd, cd = h.to(DEV, dtype), rw.to(DEV), corr.to(DEV)
    out = torch.full((M, E + extra + 2), 9.0, dtype=F32, device=DEV)
    chosen = torch.full((M, top), -1, dtype=torch.int32, device=DEV)
    p = MoeRouteParams(h=hd.data_ptr(), ldh=D, router_w=rwd.data_ptr(), correction=cd.data_ptr(), weights=out.data_ptr(), ldw=E + extra + 2, chosen=chosen.data_ptr(),
                       rows=M, D=D, E=E, top=top, n_extra=extra, score_fn=1, groups=groups, keep=keep, normalize=1, norm_eps=1e-20, scale=1.7, dtype=1 if dtype == F32 else 0)
    check(_lib.lib().evo_moe_route_ex(C.byref(p), _stream()))
    # rows whose choice rests on a close call are left out (two selection scores, or two group ranks, within 1e-4)
    c = torch.sigmoid(h.double() @ rw[:E].double().T) + corr.double()
    srt = c.sort(-1).values
    safe = (srt[:, 1:] - srt[:, :-1]).min(-1).values > 1e-4
    if groups > 1:
        per = E // groups
        rank = c.view(M, groups, per).topk(min(2, per), -1).values.sum(-1).sort(-1).values
        safe &= (rank[:, 1:] - rank[:, :-1]).min(-1).values > 1e-4
    assert safe.sum() >= M // 2
    _close(out[:, :E].cpu()[safe], want[safe], 2e-5, "weights")
    assert (out[:, E + extra:] == 9.0).all()
    picked = chosen.cpu().long()[safe].sort(-1).values
    assert torch.equal(picked, (want[safe] > 0).nonzero()[:, 1].view(-1, top))
    if extra:
        _close(out[:, E], torch.sigmoid(h.double() @ rw[E].double()), 2e-6, "the gate that rides along")


@pytest.mark.parametrize("dtype", [F32, B16])
def test_activation_kernel_erf_gelu_and_tail_weight(dtype):
    M, F, grp, E = 5, 44, 8, 4                               # 4 groups of 8 columns, then a tail of 12
    g = torch.Generator().manual_seed(2)
    z = _bf(torch.randn(M, 2 * F + 4, generator=g) * 2)
    wts = torch.rand(M, E + 1, generator=g)
    wts[:, 1] = 0.0
    zd, wd = z.to(DEV, dtype), wts.to(DEV)
    esz = zd.element_size()
    out = torch.full((M, F + 4), 7.0, dtype=dtype, device=DEV)
    lib, dt = _lib.lib(), 1 if dtype == F32 else 0
    tol = 2e-6 if dtype == F32 else 8e-3
    check(lib.evo_glu_act(ptr(zd), None, 2 * F + 4, ptr(out), F + 4, M, F, 2, None, 0, 0, 0, 0, dt, _stream()))
    _close(out[:, :F], O.gelu_erf(z[:, :F].double()), tol, "erf gelu alone")
    assert (out[:, F:] == 0).all()
    check(lib.evo_glu_act(ptr(zd), C.c_void_p(zd.data_ptr() + F * esz), 2 * F + 4, ptr(out), F + 4, M, F, 1, ptr(wd), E + 1, grp, E, 1, dt, _stream()))
    colw = torch.cat([wts[:, :E].repeat_interleave(grp, 1), wts[:, E:].expand(M, F - E * grp)], 1).double()
    _close(out[:, :F], O.silu(z[:, :F].double()) * z[:, F:2 * F].double() * colw, tol, "gated, group weights and the tail's weight")


def _attention_reference(q, k, v, scale, r1, r2, sink, pos0):
    """q (L, H, dk), k / v (pos0 + L, G, d): fp64 causal attention with distance bias and a zero-score sink."""
    L, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(L, H, v.shape[2], dtype=F64)
    for h in range(H):
        g = h // (H // G)
        for t in range(L):
            i = pos0 + t
            s = (k[:i + 1, g] @ q[t, h]) * scale
            if r1 is not None:
                s = s - r1[h] * torch.log(1 + r2[h] * (i - torch.arange(i + 1)).double())
            e = torch.exp(s - s.max())
            den = e.sum() + (torch.exp(-s.max()) if sink else 0.0)
            out[t, h] = (e / den) @ v[:i + 1, g]
    return out


@pytest.mark.parametrize("H,G,dk,dv,biased,sink,L,pos0", [(4, 2, 64, 40, True, True, 200, 0), (2, 1, 16, 16, False, False, 150, 70), (3, 1, 10, 9, True, True, 90, 37),
                                                        (6, 2, 64, 64, False, False, 130, 1), (2, 2, 128, 128, True, True, 70, 300)])
def test_attention_kernels_agree_with_bias_and_sink(H, G, dk, dv, biased, sink, L, pos0):
    """The many-query CUDA-core kernel (fp32), the tensor-core kernel (bf16, 16 rows or more) and the few-query kernel against fp64."""
    g = torch.Generator().manual_seed(H * dk + L)
    T = pos0 + L
    q, k, v = _bf(torch.randn(L, H, dk, generator=g)), _bf(torch.randn(T, G, dk, generator=g)), _bf(torch.randn(T, G, dv, generator=g))
    r1, r2 = _bf(0.3 + torch.rand(H, generator=g)), _bf(0.1 + torch.rand(H, generator=g))
    scale = 1.3 / math.sqrt(dk)
    want = _attention_reference(q.double(), k.double(), v.double(), scale, r1.double() if biased else None, r2.double(), sink, pos0).reshape(L, H * dv)
    zero = torch.zeros(H, dtype=B16, device=DEV)
    r1d, r2d = r1.to(DEV), r2.to(DEV)

    def run(dtype, rows):
        qd, kd, vd = q.to(DEV, dtype).reshape(L, H * dk), k.to(DEV, dtype).reshape(T, G * dk), v.to(DEV, dtype).reshape(T, G * dv)
        ldo = (H * dv + 63) // 64 * 64
        outs = []
        for lo in range(0, L, rows):
            n = min(rows, L - lo)
            out = torch.full((n, ldo), 5.0, dtype=dtype, device=DEV)
            p = WindowAttnParams(q=qd[lo:].data_ptr(), q_tok_stride=H * dk, k=kd.data_ptr(), v=vd.data_ptr(), k_tok_stride=G * dk, v_tok_stride=G * dv,
                                 k_batch_stride=T * G * dk, v_batch_stride=T * G * dv, out=out.data_ptr(), ldo=ldo, dtype=1 if dtype == F32 else 0, B=1, Lq=n, H=H, G=G,
                                 dk=dk, dv=dv, n_maps=1, q_pos0=pos0 + lo, scale=scale, sink=zero.data_ptr() if sink else None,
                                 dist_r1=r1d.data_ptr() if biased else None, dist_r2=r2d.data_ptr() if biased else None)
            check(_lib.lib().evo_window_attn_fwd(C.byref(p), _stream()))
            assert (out[:, H * dv:] == 0).all()
            outs.append(out[:, :H * dv])
        return torch.cat(outs, 0)
    _close(run(F32, L), want, 3e-5, "many-query kernel, fp32")
    _close(run(F32, 3), want, 3e-5, "few-query kernel, fp32")
    _close(run(B16, L), want, 1.5e-2, "tensor-core kernel")
    _close(run(B16, 2), want, 1.5e-2, "few-query kernel, bf16")


# ------------------------------------------------------------------ mixers alone: one layer without feed-forward
def _one_layer(kind, T=70, seed=0, dtype=F32, mutate=None, **sizes):
    cfg = O.make_config(layers=(kind,), mlps=(None,), **sizes)
    if mutate:
        mutate(cfg)
    W = O.random_weights(cfg, seed=seed)
    tokens = _tokens(cfg, T, seed=seed + 1)
    return cfg, W, tokens, O.forward(tokens, W, cfg), _model(cfg, W, dtype)


ATT_SIZES = [dict(att_heads=4, att_kv_heads=2, att_dim=16, rot_dims=8), dict(att_heads=3, att_kv_heads=1, att_dim=10, rot_dims=6, width=50),
             dict(att_heads=6, att_kv_heads=2, att_dim=64, rot_dims=16, width=96), dict(att_heads=2, att_kv_heads=2, att_dim=24, rot_dims=24),
             dict(att_heads=1, att_kv_heads=1, att_dim=8, rot_dims=0), dict(att_heads=2, att_kv_heads=1, att_dim=136, rot_dims=4, width=72)]


@pytest.mark.parametrize("sizes", ATT_SIZES, ids=lambda s: "h{att_heads}g{att_kv_heads}k{att_dim}r{rot_dims}".format(**s))
def test_key_valued_attention_mixer_matches_the_oracle(sizes):
    cfg, W, tokens, want, model = _one_layer("attention", T=100, seed=sizes["att_dim"], **sizes)
    got, _ = model(torch.tensor([tokens], device=DEV))
    _close(got[0], want, 3e-5, "whole")
    _close(_portions(model, tokens, [37, 2, 1, 1, 40, 19]), want, 3e-5, "portions and steps")


LEFT_SIZES = [dict(left_heads=4, left_kv_heads=2, left_dim=16, left_vdim=12, temp_every=8), dict(left_heads=3, left_kv_heads=1, left_dim=10, left_vdim=9, temp_every=3, width=50),
              dict(left_heads=2, left_kv_heads=2, left_dim=64, left_vdim=40, temp_every=0), dict(left_heads=1, left_kv_heads=1, left_dim=8, left_vdim=140, temp_every=1, width=40)]


@pytest.mark.parametrize("sizes", LEFT_SIZES, ids=lambda s: "h{left_heads}g{left_kv_heads}k{left_dim}v{left_vdim}e{temp_every}".format(**s))
def test_biased_sink_attention_side_matches_the_oracle(sizes):
    cfg, W, tokens, want, model = _one_layer("parallel", T=100, seed=sizes["left_dim"], right_scale=0.0, left_scale=1.4, **sizes)
    got, _ = model(torch.tensor([tokens], device=DEV))
    _close(got[0], want, 3e-5, "whole")
    _close(_portions(model, tokens, [37, 2, 1, 1, 40, 19]), want, 3e-5, "portions and steps")


MEM_SIZES = [dict(mem_heads=2, mem_dim=12, mem_vdim=20, gate_cap=6.0), dict(mem_heads=3, mem_dim=5, mem_vdim=7, gate_cap=2.0, width=50),
             dict(mem_heads=4, mem_dim=48, mem_vdim=40, gate_cap=10.0, width=96), dict(mem_heads=1, mem_dim=72, mem_vdim=136, gate_cap=15.0),
             dict(mem_heads=1, mem_dim=1, mem_vdim=1, gate_cap=1.0), dict(mem_heads=2, mem_dim=130, mem_vdim=31, gate_cap=5.0)]


@pytest.mark.parametrize("sizes", MEM_SIZES, ids=lambda s: "h{mem_heads}k{mem_dim}v{mem_vdim}".format(**s))
def test_matrix_memory_side_matches_the_oracle(sizes):
    cfg, W, tokens, want, model = _one_layer("parallel", T=70, seed=sizes["mem_dim"], left_scale=0.0, right_scale=0.8, **sizes)
    # gate projections large enough for the cap and the running maximum to matter
    for n in ("i", "f"):
        W[f"l0.mix.right.{n}"] = _bf(W[f"l0.mix.right.{n}"].float() * 6)
    W["l0.mix.right.i.b"] = _bf(W["l0.mix.right.i.b"].float() + 1.5)
    want = O.forward(tokens, W, cfg)
    model = _model(cfg, W)
    got, _ = model(torch.tensor([tokens], device=DEV))
    _close(got[0], want, 3e-5, "whole")
    _close(_portions(model, tokens, [1] * 70), want, 3e-5, "token by token")
    _close(_portions(model, tokens, [17, 2, 1, 33, 16, 1]), want, 3e-5, "portions that cut the kernel's rounds of 16 tokens")


def test_matrix_memory_spread_over_several_ctas_on_a_long_prompt():
    """A long prompt on few heads spreads a head's value channels over CTAs: read-outs and e^{-m} pass through the workspace."""
    cfg, W, tokens, want, model = _one_layer("parallel", T=300, seed=5, left_scale=0.0, mem_heads=1, mem_dim=16, mem_vdim=200, width=48)
    got, _ = model(torch.tensor([tokens], device=DEV))
    _close(got[0], want, 3e-5, "whole")
    _close(_portions(model, tokens, [280, 1, 1, 18]), want, 3e-5, "prompt, steps, portion")


@pytest.mark.parametrize("kind,sizes", [("delta", dict(heads=2, kv_heads=1, dim=128, vdim=72, taps=2)), ("delta", dict(heads=3, kv_heads=3, dim=66, vdim=6, taps=3)),
                                        ("parallel", dict(mem_heads=2, mem_dim=100, mem_vdim=130, left_scale=0.0)), ("parallel", dict(mem_heads=1, mem_dim=128, mem_vdim=64, left_scale=0.0))])
def test_recurrences_with_sixteen_lanes_per_column_on_a_long_prompt(kind, sizes):
    """Prompts of 256 tokens or more on few heads of 65 to 128 state rows put 16 lanes on a state column instead of 8; the portions behind the
    prompt run with 8 lanes on the state it left."""
    cfg, W, tokens, want, model = _one_layer(kind, T=300, seed=4, width=48, **sizes)
    got, _ = model(torch.tensor([tokens], device=DEV))
    _close(got[0], want, 3e-5, "whole")
    _close(_portions(model, tokens, [270, 1, 1, 28]), want, 3e-5, "prompt, steps, portion")
    _close(_portions(model, tokens, [12, 260, 28]), want, 3e-5, "a long portion on a carried state")


DELTA_SIZES = [dict(heads=4, kv_heads=2, dim=8, vdim=16, taps=3), dict(heads=3, kv_heads=1, dim=5, vdim=7, taps=2, width=50), dict(heads=6, kv_heads=3, dim=32, vdim=64, taps=4, width=96),
               dict(heads=1, kv_heads=1, dim=8, vdim=8, taps=1)]


@pytest.mark.parametrize("sizes", DELTA_SIZES, ids=lambda s: "h{heads}g{kv_heads}k{dim}v{vdim}t{taps}".format(**s))
def test_gated_delta_mixer_matches_the_oracle(sizes):
    cfg, W, tokens, want, model = _one_layer("delta", T=70, seed=sizes["dim"], **sizes)
    got, _ = model(torch.tensor([tokens], device=DEV))
    _close(got[0], want, 3e-5, "whole")
    _close(_portions(model, tokens, [1] * 70), want, 3e-5, "token by token")
    _close(_portions(model, tokens, [17, 2, 1, 33, 16, 1]), want, 3e-5, "portions")


# ------------------------------------------------------------------ keys far away, the sink, the temperature's steps
def _sharp(W, name, gain):
    W[name] = _bf(W[name].float() * gain)


@pytest.mark.parametrize("dtype", [F32, B16])
@pytest.mark.parametrize("kind", ["attention", "parallel"])
def test_far_key_among_hundreds_decides_the_answer(kind, dtype):
    """A prompt of one repeated token with ONE other token far back, under sharpened queries: rows long after it still depend on it, in
    prompts (all three attention kernels) and in steps; the model follows the oracle on both prompts."""
    cfg = O.make_config(layers=(kind,), mlps=(None,), vocab=50, right_scale=0.0, temp_every=64, rot_dims=0)
    W = O.random_weights(cfg, seed=9)
    _sharp(W, "l0.mix.left.q.norm" if kind == "parallel" else "l0.mix.q.norm", 6.0)
    if kind == "parallel":                                   # a small distance bias: the far key is not pushed out of sight
        W["l0.mix.left.r1"] = _bf(torch.full_like(W["l0.mix.left.r1"].float(), 0.3))
    T, j = 400, 5
    plain, odd = [7] * T, [7] * T
    odd[j] = 31
    want_plain, want_odd = O.forward(plain, W, cfg), O.forward(odd, W, cfg)
    rows = [j, j + 1, 130, 399]
    assert (want_odd[rows[2:]] - want_plain[rows[2:]]).abs().max() > 0.05 * want_plain.abs().max()      # the far token matters in the oracle
    model = _model(cfg, W, dtype)
    tol = 3e-5 if dtype == F32 else 4e-2
    for tokens, want in ((plain, want_plain), (odd, want_odd)):
        got, _ = model(torch.tensor([tokens], device=DEV))
        _close(got[0], want, tol, "whole")
        _close(_portions(model, tokens, [j, 2, 120, 3, 250] + [1] * (T - j - 375)), want, tol, "portions and steps")


def test_sink_takes_weight_when_every_score_is_low():
    """Scores far below zero: the zero-score sink holds almost all the weight and the attention side's output nearly vanishes."""
    cfg = O.make_config(layers=("parallel",), mlps=(None,), right_scale=0.0, temp_every=0)
    W = O.random_weights(cfg, seed=3)
    W["l0.mix.left.r1"] = _bf(torch.full_like(W["l0.mix.left.r1"].float(), 4.0))
    W["l0.mix.left.r2"] = _bf(torch.full_like(W["l0.mix.left.r2"].float(), 50.0))
    tokens = _tokens(cfg, 60)
    want = O.forward(tokens, W, cfg)
    model = _model(cfg, W)
    got, _ = model(torch.tensor([tokens], device=DEV))
    _close(got[0], want, 3e-5, "whole")
    _close(_portions(model, tokens, [30] + [1] * 30), want, 3e-5, "steps")
    first = O.forward(tokens[:1], W, cfg)                    # one token: without a sink its weight would be 1 whatever the score
    _close(got[0, :1], first, 3e-5, "first token")


def test_query_temperature_steps_at_multiples_of_its_period():
    """A large coefficient and a short period: positions p with (p + 1) a multiple of the period start a new temperature, in prompts cut
    just before, at and after such positions, and in steps."""
    cfg = O.make_config(layers=("parallel",), mlps=(None,), right_scale=0.0, temp_every=16, temp_coef=2.5)
    W = O.random_weights(cfg, seed=12)
    tokens = _tokens(cfg, 70)
    want = O.forward(tokens, W, cfg)
    flat = O.forward(tokens, W, O.make_config(layers=("parallel",), mlps=(None,), right_scale=0.0, temp_every=0))
    assert (want[15:] - flat[15:]).abs().max() > 0.05 * want.abs().max() and torch.allclose(want[:15], flat[:15])
    model = _model(cfg, W)
    got, _ = model(torch.tensor([tokens], device=DEV))
    _close(got[0], want, 3e-5, "whole")
    _close(_portions(model, tokens, [14, 1, 1, 1, 14, 2, 15, 16] + [1] * 6), want, 3e-5, "cuts around the steps")


# ------------------------------------------------------------------ the model
CONFIGS = {
    "mixed": dict(),
    "delta_first": dict(layers=("delta", "attention", "parallel", "delta", "parallel"), mlps=("moe", None, "dense", "dense", "moe"), width=72, vocab=257, rot_dims=16, temp_every=5,
                        experts=12, top=3, groups=4, keep=2, kv_heads=4),
    "bare": dict(layers=("parallel", "attention", "delta"), mlps=(None, "moe", None), rot_dims=0, temp_every=0, groups=0, shared_ff=0, taps=1, top=1),
    "ones": dict(layers=("attention", "parallel", "delta"), mlps=("moe", "moe", "dense"), att_heads=1, att_kv_heads=1, left_heads=1, left_kv_heads=1, mem_heads=1, heads=1, kv_heads=1,
                 experts=4, top=1, groups=4, keep=1, temp_every=1, left_scale=1.0, right_scale=1.0, router_scale=1.0),
    "odd": dict(layers=("delta", "parallel", "attention"), mlps=("moe", "dense", "moe"), width=50, ff=37, vocab=33, heads=3, kv_heads=1, dim=5, vdim=7, taps=2,
                att_heads=3, att_kv_heads=1, att_dim=10, rot_dims=6, left_heads=3, left_kv_heads=1, left_dim=10, left_vdim=9, temp_every=7, mem_heads=3, mem_dim=5, mem_vdim=7,
                experts=6, top=3, groups=3, keep=2, expert_ff=10, shared_ff=14),
    "wide": dict(layers=("parallel", "delta", "attention"), mlps=("moe", "dense", "dense"), width=200, ff=264, heads=2, kv_heads=2, dim=72, vdim=136, taps=4, att_heads=2, att_kv_heads=1,
                 att_dim=72, rot_dims=72, left_heads=2, left_kv_heads=1, left_dim=72, left_vdim=40, mem_heads=2, mem_dim=70, mem_vdim=136, experts=16, top=4, groups=8, keep=3,
                 expert_ff=40, shared_ff=72),
}


def _tolerance(cfg, W, tokens, want):
    """Bound on the 32-bit model's distance from the fp64 oracle: three times what the oracle itself loses when it runs in 32-bit floats
    (a deep stack can meet a nearly empty key or head output, whose norms then magnify the rounding), at least 3e-5 of the scale."""
    own = ((O.forward(tokens, W, cfg, dtype=F32).double() - want).abs().max() / want.abs().max()).item()
    assert own < 1e-4
    return max(3e-5, 3 * own)


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_model_whole_steps_and_portions_match_the_oracle_in_fp32(name):
    cfg = O.make_config(**CONFIGS[name])
    W = O.random_weights(cfg, seed=len(name))
    T = 75
    tokens = _tokens(cfg, T)
    streams = []
    want = O.forward(tokens, W, cfg, taps=streams)
    tol = _tolerance(cfg, W, tokens, want)
    model = _model(cfg, W)
    model._tap = []
    got, _ = model(torch.tensor([tokens], device=DEV))
    assert len(model._tap) == len(streams)
    for r, (a, b) in enumerate(zip(model._tap, streams)):
        _close(a, b, tol, f"{name}: stream handed on by layer {r}")
    model._tap = None
    _close(got[0], want, tol, f"{name}: whole")
    _close(_portions(model, tokens, [1] * T), want, tol, f"{name}: token by token from the first token")
    _close(_portions(model, tokens, [40] + [1] * 35), want, tol, f"{name}: prompt then steps")
    _close(_portions(model, tokens, [2, 2, 3, 30, 1, 2, 17, 9, 2, 5, 2]), want, tol, f"{name}: portions")
    _close(_portions(model, tokens[:1], [1]), want[:1], tol, f"{name}: a one-token sequence")
    _close(_portions(model, tokens[:2], [2]), want[:2], tol, f"{name}: a two-token sequence")
    model.moe_sparse_min_rows = 1                             # only the chosen experts, row by row, instead of all experts densely
    sparse, _ = model(torch.tensor([tokens], device=DEV))
    _close(sparse[0], want, tol, f"{name}: chosen experts only")


def test_layers_with_their_own_sizes_and_a_cache_that_has_to_grow():
    cfg = O.make_config(layers=("parallel", "attention", "parallel", "attention", "delta", "delta"), mlps=("moe", "dense", None, "moe", "dense", "moe"), width=104, vocab=211)
    cfg["layers"][2]["mixer"]["left"] = {"heads": 6, "kv_heads": 3, "dim": 8, "vdim": 40, "scale": 0.2}
    cfg["layers"][2]["mixer"]["right"] = {"heads": 2, "dim": 24, "vdim": 9, "gate_cap": 3.0}
    cfg["layers"][3]["mixer"] = {"heads": 2, "kv_heads": 1, "dim": 20, "vdim": 20, "scale": 0.5, "rot": {"base": 7.0, "dims": 20}}
    cfg["layers"][5]["mixer"] = {"heads": 4, "kv_heads": 4, "dim": 16, "vdim": 8, "conv": 2}
    cfg["layers"][3]["mlp"]["router"] = {"experts": 5, "top": 2, "scale": 0.7}
    cfg["layers"][3]["mlp"]["shared"] = None
    cfg["layers"][4]["mlp"]["ff"] = 72
    W = O.random_weights(cfg, seed=21)
    tokens = _tokens(cfg, 70, seed=8)
    want = O.forward(tokens, W, cfg)
    tol = _tolerance(cfg, W, tokens, want)               # six layers deep, one delta layer meets a nearly empty key
    model = _model(cfg, W)
    got, _ = model(torch.tensor([tokens], device=DEV))
    _close(got[0], want, tol, "whole")
    state = model.initialize_inference_params(max_seqlen=16, max_batch_size=1)
    _close(_portions(model, tokens, [9, 2, 20, 1, 1, 30, 7], state=state), want, tol, "portions through a growing cache")
    assert all(c.shape[1] >= 70 for c in state["mha"].key_value_memory_dict.values())


def test_model_bf16_stays_within_rounding_of_the_oracle_and_of_itself():
    cfg = O.make_config()
    W = O.random_weights(cfg, seed=3)
    tokens = _tokens(cfg, 90, seed=2)
    want = O.forward(tokens, W, cfg)
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
    none, _ = model(ids, logits_rows=[])
    assert none.shape == (0, cfg["vocab"])


def test_reused_state_memory_and_long_decoding():
    """State holders that still hold another request's rows, matrix states, running maxima and carried inputs (and NaNs beyond) serve a
    new request; decoding runs for hundreds of steps; a request interleaved with another one keeps its own state."""
    cfg = O.make_config(temp_every=32)
    W = O.random_weights(cfg, seed=7)
    model = _model(cfg, W)
    a, b = _tokens(cfg, 260, seed=6), _tokens(cfg, 60, seed=9)
    want_a, want_b = O.forward(a, W, cfg), O.forward(b, W, cfg)
    state = model.initialize_inference_params(max_seqlen=272, max_batch_size=1)
    _close(_portions(model, a, [20] + [1] * 240, state=state), want_a, 3e-5, "long decoding")
    for cache in state["mha"].key_value_memory_dict.values():
        cache[:, 100:, :3] = float("nan")
    _close(_portions(model, b, [7, 2, 51], state=state), want_b, 3e-5, "the same holders, used again from position 0")
    sa = model.initialize_inference_params(max_seqlen=128, max_batch_size=1)
    sb = model.initialize_inference_params(max_seqlen=128, max_batch_size=1)
    outs_a, outs_b = [], []
    for lo, hi in ((0, 30), (30, 31), (31, 60)):
        for tokens, st, outs in ((a, sa, outs_a), (b, sb, outs_b)):
            st["mha"].seqlen_offset = st["hyena"].seqlen_offset = lo
            lg, _ = model(torch.tensor([tokens[lo:hi]], device=DEV), inference_params_dict=st)
            outs.append(lg[0])
    _close(torch.cat(outs_a), want_a[:60], 3e-5, "interleaved a")
    _close(torch.cat(outs_b), want_b[:60], 3e-5, "interleaved b")


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
    want = O.forward(full, W, cfg)
    for s in range(n_new):                                    # each picked token is (within rounding) the oracle's argmax given the same prefix
        row = want[len(full) - n_new - 1 + s]
        assert row[picked[0, s]] >= row.max() - 2e-2, s
        _close(logits[0, s], row, 3e-5 if not device_loop else 1e-2, f"kept logits {s}")     # the device loop keeps the sampler's bf16 view of the logits


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
    want = O.forward(tokens, W, cfg)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": tokens[:25], "want": [0, 24]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": tokens[25:27], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": tokens[27:28], "want": [0]}], "end": []},
             {"step": 3, "entries": [{"id": "a", "tokens": tokens[28:], "want": [11]}], "end": ["a"]},
             {"step": 4, "entries": [{"id": "b", "tokens": tokens[:3], "want": [2]}], "end": ["b"]}]
    out = str(tmp_path / "out")
    for dtype, tol in (("float32", 3e-5), ("bfloat16", 5e-2)):
        r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", ckpt, "--dtype", dtype, "--out", out, "--max-tokens", "64"],
                           input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr
        assert [l for l in r.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(5)]
        assert not os.path.exists(os.path.join(out, "1.f32"))
        for step, rows in ((0, [0, 24]), (2, [27]), (3, [39]), (4, [2])):
            got = torch.from_numpy(np.fromfile(os.path.join(out, f"{step}.f32"), dtype="<f4").reshape(len(rows), 512).copy())
            _close(got, want[rows], tol, f"replayed step {step} in {dtype}")
