"""Host-side parts of the Fofisun path that need no GPU: configuration parsing, the order of layer runs, the registry, the cache
shapes, and the plain model's mechanisms against closed forms."""
import math

import pytest
import torch

from omchat_b200.config import ClampedMoeSpec, DiffAttentionSpec, FofisunConfig, GeluMlpSpec
from omchat_b200.model import registry
from omchat_b200.model.checkpoint import config_from_dict
from oracle import fofisun_oracle as O


def small_config():
    mix = {"conv": 4, "diff": 0.3, "dim": 12, "heads": 6, "kv_heads": 2, "mask": {"keep_first": 3, "size": 11}, "scale": 0.25, "vdim": 20}
    return {"architecture": "Fofisun", "vocab": 131, "width": 72, "norm": {"eps": 1e-5}, "loop": {"start": 1, "stop": 3, "times": 3},
            "layers": [
                {"type": "attention", "mixer": dict(mix), "mlp": {"ff": 100, "kind": "dense"}},
                {"type": "attention", "mixer": dict(mix, kv_heads=6, conv=2), "mlp": {"expert": {"ff": 28, "limit": 0.8}, "kind": "moe",
                                                                                      "router": {"experts": 5, "top": 2},
                                                                                      "shared": {"ff": 36, "limit": 1.3}}},
                {"type": "attention", "mixer": dict(mix, mask={"keep_first": 0, "size": 9}), "mlp": None},
                {"type": "attention", "mixer": dict(mix), "mlp": {"expert": {"ff": 20, "limit": 2.5}, "kind": "moe",
                                                                  "router": {"experts": 7, "top": 3}, "shared": None}}]}


def test_config_is_read_from_the_dictionary_and_round_trips():
    cfg = config_from_dict(small_config())
    assert isinstance(cfg, FofisunConfig) and cfg.vocab_size == 131 and cfg.hidden_size == 72 and cfg.norm_eps == 1e-5
    a, b, c, d = cfg.layers
    assert isinstance(a.mixer, DiffAttentionSpec) and (a.mixer.heads, a.mixer.kv_heads, a.mixer.dim, a.mixer.vdim) == (6, 2, 12, 20)
    assert a.mixer.window == 11 and a.mixer.keep_first == 3 and a.mixer.conv == 4 and a.mixer.diff == 0.3 and a.mixer.scale == 0.25
    assert isinstance(a.mlp, GeluMlpSpec) and a.mlp.ff == 100 and c.mlp is None and c.mixer.keep_first == 0 and c.mixer.window == 9
    assert isinstance(b.mlp, ClampedMoeSpec) and (b.mlp.experts, b.mlp.top, b.mlp.expert_ff, b.mlp.limit) == (5, 2, 28, 0.8)
    assert (b.mlp.shared_ff, b.mlp.shared_limit) == (36, 1.3) and d.mlp.shared_ff is None and b.mixer.kv_heads == 6
    assert (cfg.loop_start, cfg.loop_stop, cfg.loop_times) == (1, 3, 3)
    assert FofisunConfig.from_dict(cfg.to_dict()) == cfg
    assert registry.MODEL_CLASSES[FofisunConfig][1] == "FofisunForCausalLM"
    for breakage in (lambda x: x["layers"][0].update(type="something_else"), lambda x: x["layers"][0]["mixer"].update(kv_heads=4),
                     lambda x: x["layers"][1]["mlp"]["router"].update(top=6), lambda x: x["layers"][0]["mlp"].update(kind="other"),
                     lambda x: x["loop"].update(stop=9), lambda x: x["loop"].update(times=0),
                     lambda x: x["layers"][2]["mixer"]["mask"].update(size=0)):
        bad = small_config()
        breakage(bad)
        with pytest.raises(ValueError):
            config_from_dict(bad)


def test_missing_optional_entries_mean_absent_mechanisms():
    d = small_config()
    del d["loop"]
    for key in ("conv", "mask", "kv_heads"):
        del d["layers"][0]["mixer"][key]
    cfg = config_from_dict(d)
    m = cfg.layers[0].mixer
    assert m.conv == 0 and m.window is None and m.keep_first == 0 and m.kv_heads == m.heads
    assert cfg.layer_runs() == [0, 1, 2, 3]


@pytest.mark.parametrize("n,loop,want", [(6, (1, 5, 2), [0, 1, 2, 3, 4, 1, 2, 3, 4, 5]), (4, (0, 4, 3), [0, 1, 2, 3] * 3), (3, (2, 3, 1), [0, 1, 2]),
                                         (3, (1, 1, 5), [0, 1, 2]), (4, (2, 4, 2), [0, 1, 2, 3, 2, 3]), (2, (0, 1, 4), [0, 0, 0, 0, 1])])
def test_order_of_layer_runs(n, loop, want):
    d = small_config()
    d["layers"] = [d["layers"][i % 4] for i in range(n)]
    d["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    assert config_from_dict(d).layer_runs() == want
    assert O.layer_runs(n, d["loop"]) == want


def test_plain_model_visibility_and_attention_closed_forms():
    see = O.visibility(12, 4, 2)
    for i in range(12):
        for j in range(12):
            assert bool(see[i, j]) == (j <= i and (i - j < 4 or j < 2))
    assert O.visibility(5, None, 0).tolist() == torch.tril(torch.ones(5, 5)).bool().tolist()
    # equal keys: every visible value weighs the same
    T, d = 9, 4
    q, k = torch.randn(T, d, dtype=O.DT), torch.ones(T, d, dtype=O.DT)
    v = torch.arange(T, dtype=O.DT)[:, None]
    out = O.softmax_attention(q, k, v, 0.7, O.visibility(T, 3, 1))
    for i in range(T):
        js = [j for j in range(T) if j <= i and (i - j < 3 or j < 1)]
        assert math.isclose(float(out[i, 0]), sum(js) / len(js), rel_tol=1e-12)


def test_plain_model_convolution_positions_and_experts():
    x = torch.arange(1.0, 7.0, dtype=O.DT)[:, None]
    w = torch.tensor([[100.0, 10.0, 1.0]], dtype=O.DT)
    assert O.causal_conv(x, w)[:, 0].tolist() == [1.0, 12.0, 123.0, 234.0, 345.0, 456.0]
    pv = O.position_vectors(3, 6, first=4)
    assert math.isclose(float(pv[1, 2]), math.sin(5 * 10000.0 ** (-2 / 6))) and math.isclose(float(pv[1, 3]), math.cos(5 * 10000.0 ** (-2 / 6)))
    assert pv[0, 0] == math.sin(4.0) and pv[0, 1] == math.cos(4.0)
    # an expert with identity-like weights: the clamps and the shifted up branch
    h = torch.tensor([[3.0, -3.0]], dtype=O.DT)
    eye = torch.eye(2, dtype=O.DT)
    y = O.clamped_expert(h, eye, eye, eye, 2.0)
    g = [2.0, -3.0]           # the gate is clamped from above only
    u = [2.0, -2.0]           # the up branch on both sides
    for c in range(2):
        assert math.isclose(float(y[0, c]), g[c] / (1 + math.exp(-1.702 * g[c])) * (u[c] + 1.0), rel_tol=1e-12)
    assert math.isclose(O.diff_lambda(torch.tensor([1.0, 2.0]), torch.tensor([0.5, 0.25]), torch.tensor([0.0]), torch.tensor([3.0]), 0.2),
                        math.e - 1.0 + 0.2, rel_tol=1e-12)
