"""Zalunex without a GPU: configuration and registry, the spec's schedule (a stretch of layers that runs again
has a cache entry per run), tensor names, cache and state needs, refused configurations, and the plain
implementation's own consistency (the decaying sum carried by hand from one half of a sequence to the next;
the chunked form of the same sum that the kernels use for prompts; the sink as one more softmax entry)."""
import json
import math

import pytest
import torch

import plain_zalunex as plain
import zalunex_models as zm


def test_registry_finds_the_design_by_its_architecture_string(tmp_path):
    import pytorch_transformers_b200 as ptb
    from pytorch_transformers_b200.config.registry import lookup
    folder = zm.write_folder(tmp_path, "mixed")
    cfg = ptb.AutoConfig.from_pretrained(folder)
    assert isinstance(cfg, ptb.ZalunexConfig) and cfg.vocab == 211 and cfg.width == 96 and len(cfg.layers) == 3
    assert cfg.vocab_size == 211 and cfg.hidden_size == 96 and cfg.max_position_embeddings == 700
    assert lookup({"architecture": "Zalunex"}).model_type == "zalunex"
    assert lookup(cfg.to_dict()).model_type == "zalunex"
    back = ptb.ZalunexConfig.from_dict(json.loads(json.dumps(cfg.to_dict())))
    assert back.layers == cfg.layers and back.loop == cfg.loop and back.residual_mult == cfg.residual_mult


@pytest.mark.parametrize("name,runs", [("mixed", [0, 1, 2, 1, 2]), ("odd", [0, 1]), ("ones", [0, 1]), ("wide", [0, 0, 0, 1])])
def test_spec_names_every_tensor_and_gives_every_run_its_own_entry(name, runs):
    import pytorch_transformers_b200 as ptb
    from pytorch_transformers_b200.models.zalunex import zalunex_spec
    raw = zm.CONFIGS[name]
    cfg = ptb.ZalunexConfig.from_dict(raw)
    assert cfg.layer_runs() == runs == plain.layer_order(raw)
    spec = zalunex_spec(cfg)
    assert spec.stream_float32 and spec.position_table_name == "pos" and spec.max_positions == raw["max_positions"]
    assert spec.logit_softcap == float(raw["logit_softcap"] or 0.0)
    model = ptb.CausalLM(spec, cfg, device="cpu", dtype=torch.float32)
    table = model.param_table()
    want = zm.tensor_shapes(raw)
    assert set(table) == set(want)
    for tensor, (_, _, decl) in table.items():
        assert tuple(decl.shape) == tuple(want[tensor]), tensor
    assert [(e.block, e.cache_entry, e.writes_cache) for e in model.schedule] == [(b, i, True) for i, b in enumerate(runs)]
    needs = model.cache_needs()
    assert [e for e, _, _ in needs] == list(range(len(runs)))
    for (entry, c, s), b in zip(needs, runs):
        l, r = raw["layers"][b]["mixer"]["left"], raw["layers"][b]["mixer"]["right"]
        assert (c.kind, c.kv_heads, c.head_dim, c.window, c.v_head_dim) == ("window", l["kv_heads"], l["dim"], l["mask"]["size"], l["vdim"])
        assert s.numel == r["heads"] * r["dim"] * r["vdim"]
    assert model.use_graphs


def _with(name, **changes):
    cfg = json.loads(json.dumps(zm.CONFIGS[name]))
    for path, value in changes.items():
        at = cfg
        keys = path.split("__")
        for k in keys[:-1]:
            at = at[int(k)] if k.isdigit() else at[k]
        at[int(keys[-1]) if keys[-1].isdigit() else keys[-1]] = value
    return cfg


@pytest.mark.parametrize("bad", [
    _with("odd", vocab=0), _with("odd", max_positions=0), _with("odd", layers=[]), _with("odd", norm={"eps": 0}),
    _with("odd", layers__0__type="serial"),
    _with("odd", layers__0__mixer__left__kv_heads=2),                       # 5 heads on 2 K/V heads
    _with("odd", layers__0__mixer__left__mask={"size": 0}),
    _with("odd", layers__0__mixer__right__decay=[0.5]),                      # one decay for two heads
    _with("odd", layers__0__mixer__right__decay=[0.5, 1.5]),
    _with("odd", layers__0__mlp__router__top=6),                             # six of five experts
    _with("odd", layers__1__mlp__limit=0),
    _with("odd", layers__1__mlp__kind="conv"),
    _with("odd", loop={"start": 1, "stop": 3, "times": 2}),                  # beyond the last layer
    _with("odd", loop={"start": 0, "stop": 1, "times": 0}),
    _with("odd", logit_softcap=-1.0),
])
def test_configurations_that_cannot_be_built_are_refused(bad):
    import pytorch_transformers_b200 as ptb
    with pytest.raises(ptb.ConfigError):
        ptb.ZalunexConfig.from_dict(bad)


def test_parts_refuse_what_their_kernels_do_not_take():
    import pytorch_transformers_b200 as ptb
    from pytorch_transformers_b200.parts.base import BuildContext, PartSpec, make_part
    from pytorch_transformers_b200 import kernels
    build = BuildContext(torch.device("cpu"), torch.float32, kernels)
    experts = dict(hidden=8, inner=4, experts=3, top=1)
    for bad in (dict(experts, expert="plain"), dict(experts, weight_on="input"), dict(experts, score="tanh"),
                dict(experts, expert="plain", weight_on="input", identity=1, experts=2),
                dict(experts, expert="plain", weight_on="input", activation="swish")):
        with pytest.raises(ValueError):
            make_part(build, PartSpec("feed_forward", "routed_experts", bad))
    with pytest.raises(ValueError):
        make_part(build, PartSpec("mixer", "linear_attention", dict(hidden=8, heads=2, dim=4, vdim=4, decay=[0.5])))
    with pytest.raises(ValueError):
        make_part(build, PartSpec("mixer", "sink_attention", dict(hidden=8, heads=3, kv_heads=2, dim=4, vdim=4, scale=1.0)))
    attn = PartSpec("mixer", "sink_attention", dict(hidden=8, heads=2, kv_heads=1, dim=4, vdim=4, scale=1.0, window=3))
    with pytest.raises(ValueError):        # two children that both want pages
        make_part(build, PartSpec("mixer", "pair", {}, children={"left": attn, "right": attn}))
    with pytest.raises(ValueError):        # a learned position table without a float32 stream
        cfg = ptb.ZalunexConfig.from_dict(zm.CONFIGS["ones"])
        spec = ptb.models.zalunex.zalunex_spec(cfg)
        spec.stream_float32 = False
        ptb.CausalLM(spec, cfg, device="cpu", dtype=torch.float32)


def _mixer_input(cfg, seed=0, tokens=150):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(tokens, cfg["width"], generator=g, dtype=torch.float64)


def test_plain_decaying_sum_in_two_halves_equals_whole():
    cfg = zm.CONFIGS["mixed"]
    w = zm.torch_weights(cfg, 3)
    for i, layer in enumerate(cfg["layers"]):
        h = _mixer_input(cfg, i)
        m, p = layer["mixer"]["right"], f"l{i}.mix.right."
        whole, s_whole = plain.lightning_attention(h, w, p, m, 1e-5)
        first, s = plain.lightning_attention(h[:67], w, p, m, 1e-5)
        second, s_end = plain.lightning_attention(h[67:], w, p, m, 1e-5, state=s)
        torch.testing.assert_close(torch.cat([first, second]), whole, atol=1e-10, rtol=1e-9)
        torch.testing.assert_close(s_end, s_whole, atol=1e-10, rtol=1e-9)


def test_plain_decaying_sum_equals_its_chunked_form():
    """o_i = b^(i+1) S0^T q_i + sum_{s<=i} b^(i-s) (q_i . k_s) v_s within a chunk, S_end = b^n S0 + sum_s b^(n-1-s) k_s v_s^T:
    what the prompt kernels compute, here in float64 against the token-by-token definition."""
    g = torch.Generator().manual_seed(5)
    T, d, vd, b = 150, 6, 5, 0.93
    q, k, v = (torch.randn(T, n, generator=g, dtype=torch.float64) for n in (d, d, vd))
    S, ref = torch.zeros(d, vd, dtype=torch.float64), []
    for t in range(T):
        S = b * S + torch.outer(k[t], v[t])
        ref.append(S.T @ q[t])
    ref = torch.stack(ref)
    S0, out = torch.zeros(d, vd, dtype=torch.float64), []
    for c0 in range(0, T, 64):
        qc, kc, vc = q[c0:c0 + 64], k[c0:c0 + 64], v[c0:c0 + 64]
        n = qc.shape[0]
        i = torch.arange(n, dtype=torch.float64)
        lag = (i[:, None] - i[None, :]).clamp_min(0)
        A = (qc @ kc.T) * (b ** lag) * (i[:, None] >= i[None, :])
        out.append((b ** (i + 1.0))[:, None] * (qc @ S0) + A @ vc)
        S0 = b ** n * S0 + (kc * (b ** (n - 1.0 - i))[:, None]).T @ vc
    torch.testing.assert_close(torch.cat(out), ref, atol=1e-10, rtol=1e-9)
    torch.testing.assert_close(S0, S, atol=1e-10, rtol=1e-9)


def test_plain_sink_is_one_more_entry_of_the_softmax_without_a_value():
    cfg = zm.CONFIGS["odd"]
    w = zm.torch_weights(cfg, 1)
    m, p = cfg["layers"][0]["mixer"]["left"], "l0.mix.left."
    h = _mixer_input(cfg, 2, tokens=20)
    base = plain.sink_window_attention(h, w, p, m, 1e-6)
    gone = dict(w)
    gone[p + "sink"] = torch.full_like(w[p + "sink"], -1e9)           # exp(sink) = 0: an ordinary softmax
    plain_softmax = plain.sink_window_attention(h, gone, p, m, 1e-6)
    assert (base - plain_softmax).abs().max() > 1e-3
    huge = dict(w)
    huge[p + "sink"] = torch.full_like(w[p + "sink"], 60.0)           # the sink takes all the weight: nothing is read
    assert plain.sink_window_attention(h, huge, p, m, 1e-6).abs().max() < 1e-12
    # the first token sees only itself: its weight is exp(s) / (exp(s) + exp(sink))
    H, G, d, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = plain.rms((h[:1] @ w[p + "q"].T).reshape(1, H, d), 1e-6) * w[p + "q.norm"]
    k = plain.rms((h[:1] @ w[p + "k"].T).reshape(1, G, d), 1e-6) * w[p + "k.norm"]
    v = (h[:1] @ w[p + "v"].T).reshape(1, G, vd)
    s = (q[0] * k[0]).sum(-1) * m["scale"]
    weight = torch.exp(s) / (torch.exp(s) + torch.exp(w[p + "sink"]))
    first = (weight[:, None] * v[0] * torch.sigmoid(h[:1] @ w[p + "g"].T)[0][:, None]).reshape(1, -1) @ w[p + "o"].T
    torch.testing.assert_close(first, base[:1], atol=1e-10, rtol=1e-9)


def test_plain_window_sees_exactly_its_size():
    """A query whose every key but one is made invisible by the window gives that key's value."""
    cfg = zm.CONFIGS["ones"]
    w = zm.torch_weights(cfg, 1)
    m, p = cfg["layers"][0]["mixer"]["left"], "l0.mix.left."      # a window of one: every token sees itself alone
    h = _mixer_input(cfg, 3, tokens=9)
    out = plain.sink_window_attention(h, w, p, m, 1e-6)
    for t in range(9):
        alone = plain.sink_window_attention(h[t:t + 1], w, p, m, 1e-6)
        torch.testing.assert_close(out[t:t + 1], alone, atol=1e-10, rtol=1e-9)


def test_plain_expert_weight_is_on_the_input():
    cfg = zm.CONFIGS["odd"]
    w = zm.torch_weights(cfg, 2)
    mlp, p = cfg["layers"][0]["mlp"], "l0.mlp."
    h = _mixer_input(cfg, 4, tokens=6)
    ids, weights = plain.route_sigmoid(h, w, p, mlp["router"])
    assert ids.shape == (6, 3) and (weights > 0).all() and (weights < 1).all()
    assert (weights.sum(-1) - 1).abs().max() > 1e-3                  # not renormalised
    out = plain.moe_scaled_input(h, w, p, mlp)
    on_output = torch.zeros_like(h)
    for t in range(6):
        for e, s in zip(ids[t].tolist(), weights[t]):
            on_output[t] += s * (plain.gelu_erf(h[t] @ w[f"{p}e{e}.up"].T) @ w[f"{p}e{e}.down"].T)
    assert (out - on_output).abs().max() > 1e-3
    assert abs(float(plain.gelu_erf(torch.tensor(1.0, dtype=torch.float64))) - 0.5 * (1 + math.erf(1 / math.sqrt(2)))) < 1e-15
