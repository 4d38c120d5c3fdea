"""Seeded random Zalunex configurations under random cuttings of the work, against the plain implementation:
sizes drawn from the general and from the tensor-core kernels' ranges, any grouping of heads, windows from one token
to longer than the prompts, loops over any stretch of layers, layers without feed-forward; three requests as one
batch of prompts (each alone in portions, or all together), then single tokens together until each ends."""
import numpy as np
import pytest
import torch

import plain_zalunex as plain
import zalunex_models as zm
from test_zalunex_gpu import close

pytestmark = pytest.mark.gpu


def random_config(seed):
    rng = np.random.Generator(np.random.PCG64(seed))
    pick = lambda *xs: xs[int(rng.integers(len(xs)))]
    width = int(pick(40, 64, 72, 128))
    n_layers = int(rng.integers(1, 4))
    layers = []
    for _ in range(n_layers):
        kv = int(pick(1, 2, 3))
        heads = kv * int(pick(1, 2, 3, 6))
        if rng.random() < 0.5:
            dim = vdim = int(pick(64, 128))                 # the tensor-core kernels' sizes
        else:
            dim, vdim = int(pick(8, 12, 40, 96)), int(pick(8, 20, 64, 96))
        window = int(pick(1, 3, 31, 64, 65, 100, 200, 5000))
        rh = int(pick(1, 2, 5))
        if rng.random() < 0.5:
            rd, rv = int(pick(64, 128)), int(pick(64, 128))
        else:
            rd, rv = int(pick(4, 24, 40)), int(pick(4, 16, 72))
        decay = [float(pick(0.0, 0.5, 0.9, 0.97, 0.999, 1.0)) for _ in range(rh)]
        mixer = zm.pair(zm.left(heads, kv, dim, vdim, window), zm.right(rh, rd, rv, decay), float(pick(0.5, 1.0, 1.3)), float(pick(0.7, 1.0, 1.2)))
        kind = pick("dense", "moe", "moe", None)
        if kind == "dense":
            mlp = zm.dense(int(pick(24, 64, 100)), float(pick(0.5, 1.5, 7.0)))
        elif kind == "moe":
            experts = int(pick(1, 4, 7, 16))
            mlp = zm.moe(int(pick(8, 24, 64)), experts, int(rng.integers(1, min(experts, 4) + 1)))
        else:
            mlp = None
        layers.append((mixer, mlp))
    loop = None
    if rng.random() < 0.6:
        a = int(rng.integers(0, n_layers))
        b = int(rng.integers(a, n_layers + 1))
        loop = (a, b, int(rng.integers(1, 4)))
    return zm._cfg(int(pick(50, 131, 300)), width, 512, layers, float(pick(0.3, 0.5, 1.0)), float(pick(1e-5, 1e-6)),
                   pick(None, 10.0, 30.0), loop=loop)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(10))
def test_random_configuration_under_random_cutting(tmp_path, seed, dtype):
    import pytorch_transformers_b200 as ptb
    cfg = random_config(seed)
    folder = zm.write_folder(tmp_path, f"random{seed}", seed=seed, bf16=(dtype == "bfloat16"), cfg=cfg)
    model = ptb.AutoModelForCausalLM.from_pretrained(folder, dtype=dtype)
    w = zm.torch_weights(cfg, seed)
    rng = np.random.Generator(np.random.PCG64(1000 + seed))
    lengths = [int(rng.integers(1, 40)), int(rng.integers(40, 200)), int(rng.integers(200, 420))]
    reqs = zm.prompts(cfg, lengths, seed=seed)
    refs = [plain.forward(cfg, w, r) for r in reqs]
    heads = [int(rng.integers(1, n + 1)) for n in lengths]         # tokens of each request that come as its prompt
    cache = model.new_cache(64 * 12, max_slots=3)
    slots = [cache.open() for _ in reqs]
    got, want = [], []
    if rng.random() < 0.5:
        got.append(model.step(cache, slots, [r[:h] for r, h in zip(reqs, heads)], want="all"))
        want += [refs[i][:heads[i]] for i in range(3)]
    else:
        for i in range(3):                                          # each alone, in random portions
            at = 0
            while at < heads[i]:
                n = int(rng.integers(1, min(heads[i] - at, 130) + 1))
                got.append(model.step(cache, [slots[i]], [reqs[i][at:at + n]], want="all"))
                want.append(refs[i][at:at + n])
                at += n
    live, t = [i for i in range(3) if heads[i] < lengths[i]], 0
    for i in range(3):
        if heads[i] >= lengths[i]:
            cache.close(slots[i])
    while live and t < 40:
        out = model.step(cache, [slots[i] for i in live], [[reqs[i][heads[i] + t]] for i in live], want="last")
        got.append(out)
        want.append(torch.stack([refs[i][heads[i] + t] for i in live]))
        t += 1
        for i in [i for i in live if heads[i] + t >= lengths[i]]:
            cache.close(slots[i])
        live = [i for i in live if heads[i] + t < lengths[i]]
    close(torch.cat(got), torch.cat(want), dtype, f"seed {seed}: {cfg['layers'][0]['mixer']['left']}")
    model.check_errors()
    cache.check()
