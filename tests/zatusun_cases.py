"""Small Zatusun configurations for the tests (none of them a real model's sizes): odd head counts, sizes that are not multiples
of 8 or 32, grouped and ungrouped heads, chunks of 5 to 40 positions, rotations of all or part of a head with and without
interpolated frequencies, latents above and below 256 numbers, routers that take one expert of one or all of them, layers
without a feed-forward, loops at the start, in the middle, over the whole model, of one pass, and absent."""


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, base=1000.0, scaling=(4.0, 64, 8.0, 2.0), scale=None, mlp=None):
    rot = {"dims": rot_dim, "base": base}
    if scaling is not None:
        rot["scaling"] = {"factor": scaling[0], "original": scaling[1], "fast": scaling[2], "slow": scaling[3]}
    return {"type": "latent_attention", "mlp": mlp,
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "rot": rot,
                      "scale": scale if scale is not None else (dim + rot_dim) ** -0.5}}


def differential(heads, kv_heads, dim, vdim, chunk, rot_dims=None, base=500.0, scaling=(8.0, 1.0, 4.0, 32), diff=0.4, scale=None, mlp=None):
    rot = {"dims": rot_dims if rot_dims else dim, "base": base}
    if scaling is not None:
        rot["scaling"] = {"factor": scaling[0], "low": scaling[1], "high": scaling[2], "original": scaling[3]}
    return {"type": "attention", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "diff": diff, "mask": {"size": chunk}, "rot": rot,
                      "scale": scale if scale is not None else dim ** -0.5}}


def hgrn2(heads, dim, vdim, mlp=None):
    return {"type": "hgrn2", "mixer": {"heads": heads, "dim": dim, "vdim": vdim}, "mlp": mlp}


def moe(experts, top, ff, limit=1.0):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit}}


def config(layers, vocab, width, loop=None, eps=1e-5, scale=3.0, softcap=20.0, max_positions=512):
    c = {"architecture": "Zatusun", "vocab": vocab, "width": width, "max_positions": max_positions, "layers": layers, "norm": {"eps": eps},
         "embedding": {"scale": scale}, "logit_softcap": softcap}
    if loop is not None:
        c["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return c


CASES = {
    # sizes that are multiples of 8: bf16 projections run on the tensor-core GEMM; a loop of two passes in the middle; one layer
    # without a feed-forward
    "even": config([latent(4, 16, 8, 24, 32, 24, mlp=moe(6, 2, 24)), hgrn2(2, 24, 16, mlp=moe(4, 1, 16, limit=0.5)),
                    differential(4, 2, 16, 8, chunk=11, rot_dims=8, mlp=moe(6, 2, 24)), latent(2, 8, 16, 8, 40, 16, scaling=None),
                    hgrn2(4, 8, 24, mlp=moe(3, 3, 8))], vocab=120, width=64, loop=(1, 3, 2)),
    # nothing divides by 8: every projection takes the plain kernel; one head; one expert of one; no loop; ungrouped maps; a
    # rotation that leaves part of every map alone
    "odd": config([latent(3, 10, 6, 7, 20, 9, mlp=moe(1, 1, 9)), differential(3, 3, 10, 34, chunk=5, rot_dims=6, scaling=None, diff=0.8, mlp=moe(5, 3, 11, limit=2.5)),
                   hgrn2(1, 12, 10), differential(1, 1, 6, 3, chunk=64, mlp=moe(2, 2, 7))], vocab=61, width=44, eps=1e-6, scale=1.0, softcap=7.5),
    # wide heads (dim > 64, vdim > 128), a latent above 256 numbers, nine latent-attention heads (two blocks of heads), three
    # query heads per key/value head; the whole model is the loop and runs three times
    "wide": config([differential(6, 2, 40, 72, chunk=40, scaling=(16.0, 0.5, 64.0, 1000)), hgrn2(2, 72, 136, mlp=moe(4, 4, 16)),
                    latent(9, 24, 16, 40, 264, 48, base=50.0, scaling=(16.0, 32, 1000.0, 500.0))], vocab=90, width=96, loop=(0, 3, 3)),
}
