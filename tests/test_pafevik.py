"""Pafevik without a GPU: configuration and registry, the spec's schedule and tensor names, and the plain
implementation's own consistency (a sequence computed whole equals the same sequence computed with its
recurrence and cache carried from token to token by hand)."""
import json

import pytest
import torch

import pafevik_models as pm
import plain_pafevik as plain


def test_registry_finds_the_design_by_its_architecture_string(tmp_path):
    import pytorch_transformers_b200 as ptb
    from pytorch_transformers_b200.config.registry import lookup
    folder = pm.write_folder(tmp_path, "mixed")
    cfg = ptb.AutoConfig.from_pretrained(folder)
    assert isinstance(cfg, ptb.PafevikConfig) and cfg.vocab == 211 and cfg.width == 96 and len(cfg.layers) == 4
    assert cfg.vocab_size == 211 and cfg.hidden_size == 96 and not cfg.tie_word_embeddings
    assert lookup({"architecture": "Pafevik"}).model_type == "pafevik"
    assert lookup(cfg.to_dict()).model_type == "pafevik"      # a saved configuration carries model_type
    back = ptb.PafevikConfig.from_dict(json.loads(json.dumps(cfg.to_dict())))
    assert back.layers == cfg.layers and back.logit_scale == cfg.logit_scale


@pytest.mark.parametrize("name", sorted(pm.CONFIGS))
def test_spec_names_every_tensor_and_schedules_shared_entries(name):
    import pytorch_transformers_b200 as ptb
    from pytorch_transformers_b200.models.pafevik import pafevik_spec
    raw = pm.CONFIGS[name]
    cfg = ptb.PafevikConfig.from_dict(raw)
    spec = pafevik_spec(cfg)
    assert spec.stream_float32 and spec.logit_scale == raw["logit_scale"] and spec.head_name == "head"
    model = ptb.CausalLM(spec, cfg, device="cpu", dtype=torch.float32)
    table = model.param_table()
    want = pm.tensor_shapes(raw)
    assert set(table) == set(want)
    for tensor, (_, _, decl) in table.items():
        assert tuple(decl.shape) == tuple(want[tensor]), tensor
    for i, (entry, layer) in enumerate(zip(model.schedule, raw["layers"])):
        src = layer["mixer"].get("kv_from")
        assert entry.block == i and entry.cache_entry == (i if src is None else src) and entry.writes_cache == (src is None)
    needs = {e: (c, s) for e, c, s in model.cache_needs()}
    for i, layer in enumerate(raw["layers"]):
        m = layer["mixer"]
        if layer["type"] == "rglru":
            assert needs[i][0] is None and needs[i][1].numel == m["width"] * m["conv"]
        elif m.get("kv_from") is None:
            c = needs[i][0]
            assert (c.kind, c.kv_heads, c.head_dim, c.v_head_dim) == ("full", 1, m["kv_rank"] + m["rot_dim"], 0)
        else:
            assert i not in needs


@pytest.mark.parametrize("bad", [
    {"vocab": 0}, {"layers": []}, {"norm": {"eps": 0}},
    {"layers": [{"type": "conv", "mixer": {}, "mlp": None}]},
    {"layers": [dict(pm.rglru(30, 4, 2), mlp=None)]},                                  # width no multiple of blocks
    {"layers": [dict(pm.latent(2, 8, 4, 8, 8, 8, kv_from=0), mlp=None)]},                # reads itself
    {"layers": [dict(pm.latent(2, 8, 4, 8, 8, 8), mlp=None), dict(pm.latent(2, 8, 4, 8, 8, 16, kv_from=0), mlp=None)]},
    {"layers": [dict(pm.latent(2, 8, 3, 8, 8, 8), mlp=None)]},                          # odd rotated size
])
def test_configurations_that_cannot_be_built_are_refused(bad):
    import pytorch_transformers_b200 as ptb
    raw = dict(pm.CONFIGS["ones"], **bad)
    with pytest.raises(ptb.ConfigError):
        ptb.PafevikConfig.from_dict(raw)


def test_router_part_refuses_shapes_it_cannot_choose_from():
    import pytorch_transformers_b200 as ptb
    raw = json.loads(json.dumps(pm.CONFIGS["ones"]))
    raw["layers"][0]["mlp"]["router"].update(experts=4, top=3, groups={"count": 2, "keep": 1})   # 3 of 2 eligible
    cfg = ptb.PafevikConfig.from_dict(raw)
    from pytorch_transformers_b200.models.pafevik import pafevik_spec
    with pytest.raises(ValueError):
        ptb.CausalLM(pafevik_spec(cfg), cfg, device="cpu", dtype=torch.float32)


def test_plain_route_masks_groups_with_minus_infinity_not_zero():
    # all choice scores negative: an expert outside the kept group must not win with a "0"
    torch.manual_seed(0)
    h = torch.randn(5, 8, dtype=torch.float64)
    w = {"l0.mlp.router": torch.randn(6, 8, dtype=torch.float64), "l0.mlp.correction": torch.full((6,), -3.0, dtype=torch.float64)}
    router = {"experts": 6, "identity": 0, "top": 2, "scale": 1.0, "groups": {"count": 3, "keep": 1}}
    chosen, weights = plain.route(h, w, "l0.", router)
    assert ((chosen[:, 0] // 2) == (chosen[:, 1] // 2)).all()          # both from the one kept group
    s = torch.softmax(h @ w["l0.mlp.router"].T, -1)
    assert torch.allclose(weights, s.gather(1, chosen))                # weights carry no correction


def test_plain_recurrence_whole_equals_token_by_token():
    cfg = pm.CONFIGS["mixed"]
    w = pm.torch_weights(cfg, 3)
    m = cfg["layers"][1]["mixer"]
    torch.manual_seed(1)
    h = torch.randn(9, cfg["width"], dtype=torch.float64)
    whole = plain.rglru(h, w, "l1.", m)
    # by hand: the state S and the last taps - 1 inputs carried along
    R, B, K = m["width"], m["blocks"], m["conv"]
    S = torch.zeros(R, dtype=torch.float64)
    hist = torch.zeros(K - 1, R, dtype=torch.float64)
    rows = []
    for t in range(9):
        x = h[t] @ w["l1.mix.x"].T + w["l1.mix.x.b"]
        window = torch.cat([hist, x[None]])
        u = w["l1.mix.conv.b"] + (w["l1.mix.conv"].T * window).sum(0)
        hist = window[1:]
        ub = u.reshape(B, R // B)
        r = torch.sigmoid(torch.einsum("bi,boi->bo", ub, w["l1.mix.ra"]) + w["l1.mix.ra.b"]).reshape(R)
        i = torch.sigmoid(torch.einsum("bi,boi->bo", ub, w["l1.mix.ri"]) + w["l1.mix.ri.b"]).reshape(R)
        a = torch.exp(-8.0 * r * torch.nn.functional.softplus(w["l1.mix.lam"]))
        S = a * S + torch.sqrt(1 - a * a) * i * u
        y = plain.gelu_tanh(h[t] @ w["l1.mix.y"].T + w["l1.mix.y.b"])
        rows.append((S * y) @ w["l1.mix.o"].T)
    torch.testing.assert_close(torch.stack(rows), whole, atol=1e-12, rtol=1e-10)
