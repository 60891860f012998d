"""Small single-kernel drivers for ncu captures (development tool).

    ncu --set full --clock-control none -k regex:gemm_tcgen05 -c 2 -o gpurun_out/gemm python tests/harness/profile_targets.py gemm1
"""
import sys
import os
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import gpu_bringup as G

G._imports()
import torch  # noqa: E402

what = sys.argv[1]
dev = "cuda:0"
if what in ("gemm1", "gemm2"):
    variant = 1 if what == "gemm1" else 0
    M, N, K = 16384, 12288, 4096
    a = (torch.randn(M, K, device=dev) * 0.5).bfloat16(); w = (torch.randn(N, K, device=dev) / 64).bfloat16()
    bias = torch.randn(N, device=dev).bfloat16()
    for _ in range(3):
        G._gemm(a, w, M, N, K, 1, variant, bias=bias)
    torch.cuda.synchronize()
elif what == "gemm_gate":
    M, N, K = 16384, 22016, 4096
    a = (torch.randn(M, K, device=dev) * 0.5).bfloat16(); w = (torch.randn(N, K, device=dev) / 64).bfloat16()
    for _ in range(3):
        G._gemm(a, w, M, N, K, 4, 1, ldc=N // 2)
    torch.cuda.synchronize()
elif what == "hyena":
    from oracle import stripedhyena_oracle as O
    D, H, B, L = 4096, 32, 8, 8193
    cfg = O.tiny_config(num_layers=1, attn_layer_idxs=(), hidden_size=D, num_heads=H)
    sd = O.random_state_dict(cfg, seed=1)
    p = "blocks.0.filter."
    f = {"w": sd[p + "short_filter_weight"].to(dev), "b": sd[p + "short_filter_bias"].to(dev), "D": sd[p + "D"].to(dev), "p": sd[p + "poles"].to(dev), "r": sd[p + "residues"].to(dev)}
    z = torch.randn(B, L, 3 * D, device=dev).bfloat16()
    for _ in range(3):
        G._hyena_call(z, f, B, L, D, H, want_state=False)
elif what == "attn2":
    B, L, H = 2, 8193, 32
    qkv = torch.randn(B, L, 3, H, 128, device=dev).bfloat16()
    for _ in range(3):
        G._attn(qkv, B, L, H, 2)
elif what == "attn":
    B, L, H = 2, 8193, 32
    qkv = torch.randn(B, L, 3, H, 128, device=dev).bfloat16()
    for _ in range(3):
        G._attn(qkv, B, L, H, 1)
elif what == "zaverax":
    # one forward of a 2-layer Zaverax model (recurrent + attention) at width 2048: every new kernel once per forward
    from evo_b200.zaverax import Zaverax, ZaveraxConfig
    rec = {"type": "hgrn2", "mixer": {"heads": 16, "dim": 128, "vdim": 128}, "mlp": {"kind": "dense", "ff": 5464}}
    att = {"type": "attention", "mixer": {"heads": 16, "kv_heads": 16, "dim": 64, "vdim": 128, "scale": 0.125, "diff": 0.5, "mask": {"size": 1024, "keep_first": 16}},
           "mlp": {"kind": "dense", "ff": 5464}}
    zc = {"architecture": "Zaverax", "vocab": 512, "width": 2048, "layers": [rec, att], "norm": {"eps": 1e-5}, "canon": {"taps": 3},
          "loop": {"start": 0, "stop": 0, "times": 1}, "residual_mult": 0.5, "logit_softcap": 15.0}
    model = Zaverax(ZaveraxConfig.from_dict(zc)).init_random(0, device=dev)
    ids = torch.randint(0, 512, (4, 4096), device=dev)
    for _ in range(2):
        model(ids)
    torch.cuda.synchronize()
elif what in ("movalorn", "movalorn_step"):
    # a 2-layer Movalorn model (minGRU + dense feed-forward, latent attention + experts) at width 2048: one prompt of 2 x 4096 tokens
    # ("movalorn": every prompt kernel once per forward) or single-token steps of 16 sequences behind 2048 tokens ("movalorn_step")
    from evo_b200.movalorn import Movalorn, MovalornConfig
    gru = {"type": "mingru", "mixer": {"width": 2048}, "mlp": {"kind": "dense", "ff": 5632}}
    lat = {"type": "latent_attention", "mixer": {"heads": 16, "dim": 64, "rot_dim": 64, "vdim": 128, "kv_rank": 512, "scale": 0.088, "mask": {"size": 1024},
                                                 "rot": {"base": 10000.0, "dims": 64}},
           "mlp": {"kind": "moe", "expert": {"ff": 1408}, "router": {"experts": 16, "top": 4, "scale": 1.0}, "shared": {"ff": 1408}}}
    mc = {"architecture": "Movalorn", "vocab": 512, "width": 2048, "norm": {"eps": 1e-5}, "logit_scale": 1.0, "layers": [gru, lat],
          "embedding": {"scale": 1.0, "bigram": {"buckets": 4093, "mul_prev": 13, "mul_cur": 5}}}
    model = Movalorn(MovalornConfig.from_dict(mc)).init_random(0, device=dev)
    if what == "movalorn":
        ids = torch.randint(0, 512, (2, 4096), device=dev)
        for _ in range(2):
            model(ids)
    else:
        B, ctx = 16, 2048
        d = model.initialize_inference_params(max_seqlen=ctx + 64, max_batch_size=B)
        lg, d = model(torch.randint(0, 512, (B, ctx), device=dev), inference_params_dict=d)
        nxt = lg[:, -1].argmax(-1, keepdim=True)
        for t in range(3):
            d["mha"].seqlen_offset = d["hyena"].seqlen_offset = ctx + t
            lg, _ = model(nxt, inference_params_dict=d)
    torch.cuda.synchronize()
elif what in ("nelovik", "nelovik_step"):
    # a 2-layer Nelovik model (gated delta rule; pooled-window attention beside a state-space mixer) at width 2048: one prompt of
    # 2 x 4096 tokens ("nelovik": every prompt kernel once per forward) or single-token steps of 16 sequences behind 2048 tokens
    from evo_b200.nelovik import Nelovik, NelovikConfig
    mlp = {"kind": "dense", "ff": 5632}
    delta = {"type": "delta", "mixer": {"heads": 16, "kv_heads": 16, "dim": 128, "vdim": 128, "conv": 4}, "mlp": mlp}
    par = {"type": "parallel", "mlp": mlp, "mixer": {
        "left": {"heads": 16, "kv_heads": 16, "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "softcap": 30.0, "mask": {"size": 1024, "pool": 64},
                 "rot": {"dims": 64, "base": 10000.0}},
        "right": {"heads": 32, "vdim": 64, "state": 128, "groups": 8, "norm_groups": 8, "conv": 4}}}
    nc = {"architecture": "Nelovik", "vocab": 512, "width": 2048, "norm": {"eps": 1e-5}, "layers": [delta, par]}
    model = Nelovik(NelovikConfig.from_dict(nc)).init_random(0, device=dev)
    if what == "nelovik":
        ids = torch.randint(0, 512, (2, 4096), device=dev)
        for _ in range(2):
            model(ids)
    else:
        B, ctx = 16, 2048
        d = model.initialize_inference_params(max_seqlen=ctx + 64, max_batch_size=B)
        lg, d = model(torch.randint(0, 512, (B, ctx), device=dev), inference_params_dict=d)
        nxt = lg[:, -1].argmax(-1, keepdim=True)
        for t in range(3):
            d["mha"].seqlen_offset = d["hyena"].seqlen_offset = ctx + t
            lg, _ = model(nxt, inference_params_dict=d)
    torch.cuda.synchronize()
elif what in ("gakupel", "gakupel_step"):
    # a 2-layer Gakupel model (biased sink attention beside a matrix memory; key-valued attention; one dense and one expert feed-forward) at
    # width 2048: one prompt of 2 x 4096 tokens ("gakupel": every prompt kernel once per forward) or single-token steps of 16 sequences
    from evo_b200.gakupel import Gakupel, GakupelConfig
    moe = {"kind": "moe", "expert": {"ff": 1408}, "router": {"experts": 16, "top": 4, "scale": 2.5, "groups": {"count": 4, "keep": 2}}, "shared": {"ff": 1408}}
    par = {"type": "parallel", "mlp": moe, "mixer": {
        "left": {"heads": 16, "kv_heads": 4, "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "q_temp": {"coef": 0.25, "every": 512}}, "left_scale": 1.0,
        "right": {"heads": 16, "dim": 128, "vdim": 128, "gate_cap": 15.0}, "right_scale": 1.0}}
    att = {"type": "attention", "mlp": {"kind": "dense", "ff": 5632},
           "mixer": {"heads": 16, "kv_heads": 8, "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "rot": {"dims": 64, "base": 10000.0}}}
    gc = {"architecture": "Gakupel", "vocab": 512, "width": 2048, "norm": {"eps": 1e-5}, "layers": [par, att]}
    model = Gakupel(GakupelConfig.from_dict(gc)).init_random(0, device=dev)
    if what == "gakupel":
        ids = torch.randint(0, 512, (2, 4096), device=dev)
        for _ in range(2):
            model(ids)
    else:
        B, ctx = 16, 2048
        d = model.initialize_inference_params(max_seqlen=ctx + 64, max_batch_size=B)
        lg, d = model(torch.randint(0, 512, (B, ctx), device=dev), inference_params_dict=d)
        nxt = lg[:, -1].argmax(-1, keepdim=True)
        for t in range(3):
            d["mha"].seqlen_offset = d["hyena"].seqlen_offset = ctx + t
            lg, _ = model(nxt, inference_params_dict=d)
    torch.cuda.synchronize()
print("done", what)
