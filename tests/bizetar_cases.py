"""Small Bizetar configurations for the tests (none of them a real model's sizes): odd head counts, sizes that are not
multiples of 8 or 32, grouped and ungrouped heads, convolutions of 1 to 5 taps, rotations of all or part of a head with and
without interpolated frequencies, routers that take one expert or all of them with and without identity experts, layers
without a feed-forward, value mixing that starts at the first layer, later, or never."""


def attention(heads, kv_heads, dim, vdim, scale=None, q_temp=(0.5, 7), v_mix=False, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5}
    if q_temp is not None:
        m["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    if v_mix:
        m["v_mix"] = True
    return {"type": "attention", "mixer": m, "mlp": mlp}


def attention_2(heads, kv_heads, dim, vdim, conv=3, rot_dims=None, base=1000.0, scaling=(4.0, 64, 8.0, 2.0), scale=None, v_mix=False, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5}
    if conv:
        m["conv"] = conv
    if rot_dims:
        m["rot"] = {"dims": rot_dims, "base": base}
        if scaling is not None:
            m["rot"]["scaling"] = {"factor": scaling[0], "original": scaling[1], "fast": scaling[2], "slow": scaling[3]}
    if v_mix:
        m["v_mix"] = True
    return {"type": "attention_2", "mixer": m, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, identity=0):
    return {"kind": "moe", "router": {"experts": experts, "top": top, "identity": identity}, "expert": {"ff": ff}}


def config(layers, vocab, width, eps=1e-5):
    return {"architecture": "Bizetar", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": eps}}


CASES = {
    # sizes that are multiples of 8: bf16 projections run on the tensor-core GEMM; values mixed from the second layer on
    "even": config([attention_2(4, 2, 16, 24, conv=4, rot_dims=16, mlp=dense(72)),
                    attention(6, 2, 24, 16, v_mix=True, mlp=moe(6, 2, 24, identity=2)),
                    attention_2(4, 4, 24, 8, conv=2, rot_dims=8, scaling=None, v_mix=True, mlp=moe(4, 4, 16)),
                    attention(2, 1, 40, 32, q_temp=(1.5, 1), v_mix=True, mlp=dense(40)),
                    attention_2(8, 1, 8, 32, conv=3, rot_dims=8, v_mix=True)], vocab=120, width=64),
    # nothing divides by 8: every projection takes the plain kernel; one head, no convolution, one expert of one, a router
    # whose only other output is an identity expert; no layer mixes values
    "odd": config([attention(1, 1, 12, 10, mlp=moe(1, 1, 9, identity=1)), attention_2(3, 1, 10, 7, conv=None, rot_dims=6, mlp=dense(30)),
                   attention_2(3, 3, 12, 34, conv=5, rot_dims=None, mlp=moe(5, 3, 11, identity=3)), attention(5, 5, 6, 3, q_temp=None)],
                  vocab=61, width=44, eps=1e-6),
    # wide heads (dim > 64, vdim > 64), nine query heads on three key/value heads, value mixing from the first layer, a
    # rotation that covers part of a head with all frequencies but the first interpolated
    "wide": config([attention(9, 3, 72, 40, v_mix=True), attention_2(3, 3, 80, 40, conv=2, rot_dims=34, base=50.0, scaling=(16.0, 32, 1000.0, 500.0), v_mix=True, mlp=dense(16)),
                    attention_2(2, 1, 136, 120, conv=3, rot_dims=136, v_mix=True)], vocab=90, width=96),
}
