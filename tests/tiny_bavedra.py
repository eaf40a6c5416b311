"""Tiny Bavedra configurations for the tests: they differ in every size, constant and layer order."""

import os

import torch


def rglru(width, blocks, conv, mlp, **more):
    return dict(type="rglru", mixer=dict(width=width, blocks=blocks, conv=conv), mlp=mlp, **more)


def delta(heads, kv_heads, dim, vdim, conv, mlp, **more):
    return dict(type="delta", mixer=dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=conv), mlp=mlp, **more)


def left(heads, kv_heads, dim, scale, window=None, rot=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, scale=scale)
    if window is not None:
        m["mask"] = dict(size=window)
    if rot is not None:
        m["rot"] = dict(base=rot[0], dims=rot[1])
    return m


def right(heads, vdim, state, groups, conv, norm_groups):
    return dict(heads=heads, vdim=vdim, state=state, groups=groups, conv=conv, norm_groups=norm_groups)


def parallel(left_side, right_side, mlp, **more):
    return dict(type="parallel", mixer=dict(left=left_side, right=right_side), mlp=mlp, **more)


def dense(ff):
    return dict(kind="dense", ff=ff)


def moe(experts, top, ff, identity=None, groups=None, shared=None):
    router = dict(experts=experts, top=top)
    if identity is not None:
        router["identity"] = identity
    if groups is not None:
        router["groups"] = dict(count=groups[0], keep=groups[1])
    out = dict(kind="moe", expert=dict(ff=ff), router=router)
    if shared is not None:
        out["shared"] = dict(ff=shared)
    return out


def again(layer, source):
    out = dict(layer)
    out["weights_of"] = source
    return out


# the recurrent unit first with three blocks and three taps; a window of 10 with half of each head rotated, three
# state-space heads in three norm groups with two taps; two of three groups of router outputs with one identity
# expert; a delta layer without a feed-forward that runs twice, the second time far from the first; a window longer
# than any test sequence
_A2 = delta(4, 2, 12, 8, 4, None)
B_A = dict(architecture="Bavedra", vocab=200, width=64, embedding=dict(scale=2.0), norm=dict(eps=1e-5), layers=[
    rglru(96, 3, 3, dense(80)),
    parallel(left(4, 2, 16, 0.3, 10, (100.0, 8)), right(3, 8, 12, 1, 2, 3), moe(5, 2, 24, identity=1, groups=(3, 2), shared=16)),
    _A2,
    parallel(left(2, 2, 8, 0.4, 500, (50.0, 2)), right(1, 24, 5, 1, 4, 1), dense(48)),
    again(_A2, 2),
])

# one delta head of sizes that are no powers of two, run twice in a row, all three of three experts, no identity
# experts, groups or shared expert; one attention head, rotated as a whole, with a window of 3; state-space heads in
# two groups with a state of 33; a recurrent unit of one block; one expert of four and two identity experts
_B0 = delta(1, 1, 40, 24, 2, moe(3, 3, 32))
B_B = dict(architecture="Bavedra", vocab=131, width=96, embedding=dict(scale=1.0), norm=dict(eps=1e-6), layers=[
    _B0,
    again(_B0, 0),
    parallel(left(1, 1, 24, 0.2, 3, (10000.0, 24)), right(2, 20, 33, 2, 4, 1), dense(64)),
    rglru(64, 1, 4, moe(4, 1, 16, identity=2, groups=(2, 1), shared=8)),
])

# sizes the tensor-core kernels take: attention heads of 64 and 32 with windows of 65 and 64 around a page border,
# four query heads a key/value head and one, an attention without rotation; as many identity experts as experts;
# state-space states of 64 and 128; a delta head of 128 x 64
B_C = dict(architecture="Bavedra", vocab=257, width=128, embedding=dict(scale=11.0), norm=dict(eps=1e-5), layers=[
    parallel(left(8, 2, 64, 0.11, 65, (10000.0, 32)), right(4, 32, 64, 2, 4, 2),
             moe(8, 2, 64, identity=8, groups=(4, 2), shared=64)),
    rglru(128, 2, 4, dense(192)),
    parallel(left(4, 4, 32, 0.18, 64), right(2, 64, 128, 1, 3, 4), None),
    delta(2, 2, 128, 64, 4, moe(8, 3, 32, groups=(2, 1))),
])

TINY_B = {"BA": B_A, "BB": B_B, "BC": B_C}


def random_config(rng):
    """A configuration drawn from ``rng`` (a ``random.Random``): two to six layers of any kind in any order, some
    of them running an earlier layer's weights, with sizes, head counts, windows, taps, groups and constants drawn
    anew for every layer."""
    def feed_forward():
        kind = rng.random()
        if kind < 0.2:
            return None
        if kind < 0.45:
            return dense(rng.choice([40, 64, 96, 136, 256]))
        experts, identity = rng.choice([2, 3, 4, 6, 8, 12]), rng.choice([0, 0, 1, 2, 4])
        outputs = experts + identity
        count = rng.choice([c for c in (1, 2, 3, 4, 6) if outputs % c == 0])
        keep = rng.randint(1, count)
        top = rng.randint(1, min(outputs // count * keep, 4))
        return moe(experts, top, rng.choice([16, 24, 32, 48, 64]), identity=identity if identity or rng.random() < 0.3 else None,
                   groups=(count, keep) if count > 1 or rng.random() < 0.5 else None,
                   shared=rng.choice([16, 40, 64, 96]) if rng.random() < 0.6 else None)

    def layer():
        kind = rng.choice(["rglru", "parallel", "delta"])
        if kind == "rglru":
            blocks = rng.choice([1, 2, 4])
            return rglru(blocks * rng.choice([8, 16, 24, 32, 64]), blocks, rng.choice([2, 3, 4]), feed_forward())
        if kind == "delta":
            kv = rng.choice([1, 2, 4])
            return delta(kv * rng.choice([1, 2]), kv, rng.choice([8, 16, 24, 32, 64, 128]), rng.choice([8, 16, 32, 48, 64]),
                         rng.choice([2, 3, 4]), feed_forward())
        kv, dim = rng.choice([1, 2, 4]), rng.choice([8, 16, 32, 64, 128])
        attention = left(kv * rng.choice([1, 2, 4]), kv, dim, rng.choice([dim ** -0.5, 0.2, 0.1]),
                         rng.choice([1, 2, 5, 17, 40, 64, 65, 100, 300]),
                         (rng.choice([100.0, 1e4, 1e6]), rng.choice([d for d in (2, 4, 8, 16, 32, 64, 128) if d <= dim])))
        groups = rng.choice([1, 2])
        heads, vdim = groups * rng.choice([1, 2, 3]), rng.choice([8, 16, 24, 48, 64])
        recurrence = right(heads, vdim, rng.choice([4, 16, 32, 48, 64, 128]), groups, rng.choice([2, 3, 4]),
                           rng.choice([n for n in (1, 2, 3, 4) if (heads * vdim) % n == 0]))
        return parallel(attention, recurrence, feed_forward())

    layers = []
    for _ in range(rng.randint(2, 6)):
        own = [j for j, made in enumerate(layers) if "weights_of" not in made]
        if own and rng.random() < 0.2:
            source = rng.choice(own)
            layers.append(again(layers[source], source))
        else:
            layers.append(layer())
    return dict(architecture="Bavedra", vocab=rng.choice([97, 200, 333, 500, 1000]), width=rng.choice([48, 64, 72, 96, 128, 160, 256]),
                embedding=dict(scale=rng.choice([1.0, 2.5, 4.0, 8.0])), norm=dict(eps=rng.choice([1e-6, 1e-5])), layers=layers)


def make_bavedra_folder(tmp_path, name, seed=0, dtype=torch.float32, raw=None):
    """A model folder of the tiny configuration ``name`` (or of ``raw``, a configuration given as it is)."""
    from starter_b200.config import config_from_dict
    from starter_b200.weights import write_model_folder

    raw = TINY_B[name] if raw is None else raw
    path = os.path.join(str(tmp_path), f"tiny_{name}_{seed}")
    write_model_folder(path, config_from_dict(raw), seed, dtype)
    # The library draws matrices from N(0, 0.02): with those every score is near 0, every softmax near uniform,
    # every decay the same and every gate a half, and a wrong key, a lost state or a window that is one token off
    # would hardly show.  Larger matrices give scores of order one and routers that decide; decay constants spread
    # from short to long memory.
    from safetensors.torch import load_file, save_file

    file = os.path.join(path, "model.safetensors")
    tensors = load_file(file)
    for key, value in tensors.items():
        v = value.float()
        if key == "embed":
            v = v * (100.0 / raw["embedding"]["scale"])
        elif key.endswith((".left.q", ".left.k")):
            v = v * 14.0
        elif key.endswith(".router"):
            v = v * 40.0
        elif key.endswith(".correction"):
            v = v * 3.0
        elif key.endswith(".lam"):
            v = torch.linspace(-6.0, 1.0, v.numel()).reshape(v.shape) + v
        elif key.endswith(".A_log"):
            v = torch.linspace(-4.0, 0.5, v.numel()).reshape(v.shape) + v
        elif key.endswith(".D"):
            v = 1.0 + 3.0 * v
        elif key.endswith((".conv", ".q.conv", ".k.conv", ".v.conv")):
            v = v * 5.0
        elif key.endswith((".ra", ".ri")):
            v = v * 10.0
        elif value.dim() == 2:
            v = v * 5.0
        elif key.endswith(".b"):
            v = v * 10.0
        tensors[key] = v.to(value.dtype)
    save_file(tensors, file, metadata={"format": "pt"})
    return path
