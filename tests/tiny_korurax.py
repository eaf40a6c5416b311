"""Tiny Korurax configurations for the tests: they differ in every size, constant and layer order."""

import os

import torch


def attention(heads, kv_heads, dim, vdim, scale, chunk, mlp):
    return dict(type="attention", mixer=dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale,
                                             mask=dict(size=chunk)), mlp=mlp)


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base, mlp, dims=None):
    return dict(type="latent_attention", mlp=mlp,
                mixer=dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, q_rank=q_rank, kv_rank=kv_rank, scale=scale,
                           rot=dict(base=base, dims=rot_dim if dims is None else dims)))


def dense(ff, limit):
    return dict(kind="dense", ff=ff, limit=limit)


def moe(experts, top, ff, scale):
    return dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top, scale=scale))


# attention first; chunks of 10 and of exactly a page; values longer and shorter than keys; a layer without a
# feed-forward; all three of three experts; experts of 24 (no multiple of 16)
R_A = dict(architecture="Korurax", vocab=200, width=64, norm=dict(eps=1e-5), residual_mult=0.5, logit_softcap=30.0, layers=[
    attention(4, 2, 16, 32, 0.25, 10, moe(5, 2, 24, 2.0)),
    latent(3, 16, 8, 24, 24, 32, 0.2, 100.0, dense(96, 1.5)),
    attention(2, 2, 8, 8, 0.35, 64, None),
    latent(2, 8, 8, 16, 16, 32, 0.3, 100.0, moe(3, 3, 16, 1.0)),
])

# latent attention first, one head, only half of the rotated part turned; chunks of 3, of 65 and longer than any
# test sequence; six query heads on one key/value head; head sizes the tensor-core kernels do not take; one
# expert of three; a multiplier of one; an odd vocabulary; a cap the logits reach
R_B = dict(architecture="Korurax", vocab=131, width=96, norm=dict(eps=1e-6), residual_mult=1.0, logit_softcap=4.0, layers=[
    latent(1, 24, 16, 8, 40, 48, 0.15, 10000.0, moe(3, 1, 32, 0.7), dims=8),
    attention(6, 1, 24, 40, 0.2, 3, dense(80, 0.6)),
    attention(3, 3, 16, 16, 0.25, 500, None),
    latent(5, 8, 4, 8, 8, 16, 0.35, 50.0, None),
    attention(2, 1, 32, 16, 0.18, 65, moe(4, 2, 16, 1.5)),
])

# sizes the tensor-core tiles take (the second attention layer's also the tcgen05 prompt kernel's); three and
# eight query heads a key/value head; chunks of 64, 100 and 130
R_C = dict(architecture="Korurax", vocab=257, width=128, norm=dict(eps=1e-5), residual_mult=0.25, logit_softcap=12.0, layers=[
    attention(4, 2, 32, 64, 0.18, 64, dense(192, 2.0)),
    latent(4, 32, 32, 32, 64, 64, 0.125, 10000.0, moe(8, 2, 64, 2.5)),
    attention(6, 2, 64, 64, 0.125, 100, moe(8, 3, 32, 1.0)),
    attention(8, 1, 16, 16, 0.25, 130, dense(64, 1.0)),
])

# wider, for prompts of hundreds of tokens: keys and values of 128 (the tcgen05 prompt kernel at its larger head
# size), few experts (hundreds of rows an expert: the grouped tcgen05 product) next to more (the 128-row tiles),
# a latent of 256 with a rotated part of 32, chunks of 300 and 97
R_D = dict(architecture="Korurax", vocab=500, width=320, norm=dict(eps=1e-5), residual_mult=0.4, logit_softcap=80.0, layers=[
    attention(8, 2, 128, 128, 0.09, 300, moe(4, 2, 128, 1.5)),
    latent(8, 64, 32, 64, 96, 256, 0.1, 500000.0, dense(640, 3.0)),
    attention(4, 4, 64, 64, 0.11, 97, moe(8, 2, 80, 2.0)),
    latent(2, 48, 16, 32, 64, 64, 0.125, 10000.0, None),
])

TINY_R = {"RA": R_A, "RB": R_B, "RC": R_C, "RD": R_D}


def make_korurax_folder(tmp_path, name, seed=0, dtype=torch.float32):
    from starter_b200.config import config_from_dict
    from starter_b200.weights import write_model_folder

    path = os.path.join(str(tmp_path), f"tiny_{name}_{seed}")
    write_model_folder(path, config_from_dict(TINY_R[name]), seed, dtype)
    # The library draws matrices from N(0, 0.02): with those every score is near 0, every softmax near
    # uniform, every clamp idle and the sink and the penalty would outweigh all keys; a wrong key or a chunk
    # that is one token off would hardly show.  Larger matrices give scores of order one, feed-forwards that
    # reach their limits and routers that decide; penalties, sinks and depth weights are spread.
    from safetensors.torch import load_file, save_file

    file = os.path.join(path, "model.safetensors")
    tensors = load_file(file)
    gen = torch.Generator().manual_seed(1000 + seed)
    for key, value in tensors.items():
        v = value.float()
        if key == "embed":
            v = v * 50.0
        elif key.endswith((".uq", ".uk", ".mix.q", ".mix.k")):
            v = v * 10.0
        elif key.endswith(".router"):
            v = v * 30.0
        elif key.endswith(".mix.g"):
            v = v * 20.0
        elif key.endswith(".r1"):
            v = torch.rand(v.shape, generator=gen) * 0.8 + 0.05
        elif key.endswith(".r2"):
            v = torch.rand(v.shape, generator=gen) * 1.5 + 0.05
        elif key.endswith(".sink"):
            v = torch.randn(v.shape, generator=gen)
        elif key.endswith(".dwa"):
            v = torch.rand(v.shape, generator=gen) * 0.9 + 0.1
        elif value.dim() == 2:
            v = v * 4.0
        tensors[key] = v.to(value.dtype)
    save_file(tensors, file, metadata={"format": "pt"})
    return path
