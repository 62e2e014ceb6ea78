"""Host-side parts of the Vefunex path that need no GPU: configuration parsing and its refusals, the registry, cache and state
shapes, weight names and shapes, and the plain model's mechanisms against closed forms."""
import math

import pytest
import torch

from omchat_b200.config import (AttentionScanMixerSpec, GatedLinearAttentionSpec, SigmoidMoeSpec, SoftmaxAttentionSpec, VefunexConfig)
from omchat_b200.model import registry
from omchat_b200.model.checkpoint import config_from_dict
from oracle import vefunex_oracle as O

F64 = torch.float64


def small_config():
    moe = {"expert": {"ff": 28}, "kind": "moe", "router": {"experts": 5, "top": 2}}
    return {"architecture": "Vefunex", "vocab": 131, "width": 72, "norm": {"eps": 1e-5}, "residual_mult": 0.4, "logit_softcap": 12.0,
            "canon": {"taps": 4}, "layers": [
                {"type": "parallel", "mixer": {"left": {"dim": 12, "heads": 6, "kv_heads": 2, "rot": {"base": 5000.0, "dims": 8}, "scale": 0.25,
                                                        "softcap": 8.0, "vdim": 20}, "left_scale": 1.3, "right_scale": 0.7,
                                               "right": {"conv": 3, "dt_rank": 3, "inner": 40, "state": 5}}, "mlp": dict(moe)},
                {"type": "attention", "mixer": {"dim": 24, "heads": 4, "kv_heads": 4, "q_temp": {"coef": 0.5, "every": 7}, "scale": 0.2, "vdim": 8},
                 "mlp": None},
                {"type": "gla", "mixer": {"dim": 20, "heads": 3, "tau": 9.0, "vdim": 12}, "mlp": dict(moe, router={"experts": 7, "top": 3})}]}


def test_config_is_read_from_the_dictionary_and_round_trips():
    cfg = config_from_dict(small_config())
    assert isinstance(cfg, VefunexConfig) and (cfg.vocab_size, cfg.hidden_size, cfg.norm_eps) == (131, 72, 1e-5)
    assert (cfg.residual_mult, cfg.logit_softcap, cfg.canon_taps) == (0.4, 12.0, 4)
    a, b, c = cfg.layers
    assert isinstance(a.mixer, AttentionScanMixerSpec) and (a.mixer.left_scale, a.mixer.right_scale) == (1.3, 0.7)
    L, R = a.mixer.left, a.mixer.right
    assert isinstance(L, SoftmaxAttentionSpec) and (L.heads, L.kv_heads, L.dim, L.vdim, L.scale, L.softcap) == (6, 2, 12, 20, 0.25, 8.0)
    assert (L.rot.dims, L.rot.base) == (8, 5000.0) and L.sink and L.gate and not L.value_norm and L.q_temp_coef == 0.0
    assert (R.inner, R.state, R.dt_rank, R.conv) == (40, 5, 3, 3)
    assert isinstance(b.mixer, SoftmaxAttentionSpec) and b.mixer.value_norm and not b.mixer.sink and not b.mixer.gate and b.mixer.rot is None
    assert (b.mixer.q_temp_coef, b.mixer.q_temp_every) == (0.5, 7) and b.mlp is None
    assert isinstance(c.mixer, GatedLinearAttentionSpec) and (c.mixer.heads, c.mixer.dim, c.mixer.vdim, c.mixer.tau) == (3, 20, 12, 9.0)
    assert isinstance(a.mlp, SigmoidMoeSpec) and (a.mlp.experts, a.mlp.top, a.mlp.expert_ff) == (5, 2, 28) and c.mlp.top == 3
    assert VefunexConfig.from_dict(cfg.to_dict()) == cfg
    assert registry.MODEL_CLASSES[VefunexConfig][1] == "VefunexForCausalLM"
    for breakage in (lambda x: x["layers"][0].update(type="something_else"), lambda x: x["layers"][0]["mixer"]["left"].update(kv_heads=4),
                     lambda x: x["layers"][0]["mlp"]["router"].update(top=6), lambda x: x["layers"][0]["mlp"].update(kind="dense"),
                     lambda x: x["layers"][0]["mixer"]["left"]["rot"].update(dims=7), lambda x: x["layers"][0]["mixer"]["left"]["rot"].update(dims=14),
                     lambda x: x["layers"][2]["mixer"].update(tau=0.0), lambda x: x["canon"].update(taps=0),
                     lambda x: x["layers"][1]["mixer"]["q_temp"].update(every=0), lambda x: x["layers"][0]["mixer"]["right"].update(state=0)):
        bad = small_config()
        breakage(bad)
        with pytest.raises(ValueError):
            config_from_dict(bad)


def test_missing_optional_entries_mean_absent_mechanisms():
    d = small_config()
    del d["canon"], d["logit_softcap"], d["residual_mult"]
    del d["layers"][0]["mixer"]["left"]["rot"], d["layers"][0]["mixer"]["left"]["softcap"], d["layers"][0]["mixer"]["left"]["kv_heads"]
    del d["layers"][1]["mixer"]["q_temp"]
    cfg = config_from_dict(d)
    L = cfg.layers[0].mixer.left
    assert cfg.canon_taps == 1 and cfg.logit_softcap == 0.0 and cfg.residual_mult == 1.0
    assert L.rot is None and L.softcap == 0.0 and L.kv_heads == L.heads and cfg.layers[1].mixer.q_temp_coef == 0.0


def test_weights_names_shapes_and_state_layout():
    """random_state_dict writes what weights_from_state_dict reads; shapes that contradict the config are refused; the decoder's
    cache widths and state shapes follow the config."""
    from omchat_b200.model.vefunex import VefunexDecoder, random_state_dict, weights_from_state_dict
    cfg = config_from_dict(small_config())
    sd = random_state_dict(cfg, seed=1)
    w = weights_from_state_dict(sd, cfg, "cpu", torch.float32)
    assert w.layers[0].mix.left.w_in.shape == (6 * 12 + 2 * 12 + 2 * 20 + 6 * 20 + 2 * 40, 72) and w.layers[0].mix.left.cols["rin"] == slice(256, 336)
    assert w.layers[0].mix.right.x_dt.shape == (8, 40) and w.layers[0].mix.right.x_bc.shape == (16, 40)   # 3 and 2 * 5 rows, padded to multiples of 8
    assert w.layers[2].mix.w_in.shape[0] % 8 == 0 and w.layers[2].mix.a1.shape == (16, 72) and w.layers[0].mlp.gate_up.shape == (5, 56, 72) and w.layers[1].mlp is None
    assert [l.dwa.numel() for l in w.layers] == [2, 3, 4] and w.layers[0].norm1.alpha.dtype == torch.float32
    dec = VefunexDecoder.__new__(VefunexDecoder)
    dec.cfg, dec.C = cfg, 72
    assert dec.cache_widths() == [2 * (12 + 20), 4 * (24 + 8), 0]
    assert dec.state_shapes() == [{"canon1": (3, 72), "canon2": (3, 72), "S": (40, 5), "conv": (2, 40)}, {"canon1": (3, 72)},
                                  {"canon1": (3, 72), "canon2": (3, 72), "S": (3, 20, 12)}]
    bad = dict(sd)
    bad["l0.mix.right.A_log"] = sd["l0.mix.right.A_log"][:, :4]
    with pytest.raises(ValueError):
        weights_from_state_dict(bad, cfg, "cpu", torch.float32)
    bad = dict(sd)
    del bad["l0.mix.left.sink"]
    with pytest.raises(KeyError):
        weights_from_state_dict(bad, cfg, "cpu", torch.float32)


def test_oracle_pieces_against_closed_forms():
    # tanh norm: large alpha saturates to +-w + b
    x = torch.tensor([[-3.0, 0.0, 5.0]], dtype=F64)
    y = O.dyt(x, torch.tensor([2.0, 2.0, 2.0]), torch.tensor([0.5, 0.5, 0.5]), torch.tensor(50.0))
    assert torch.allclose(y, torch.tensor([[-1.5, 0.5, 2.5]], dtype=F64))
    # convolution: the last tap multiplies the token itself, the first the one taps - 1 back; zeros before the start
    h = torch.arange(1, 6, dtype=F64)[:, None]
    w = torch.tensor([[100.0, 10.0, 1.0]], dtype=F64)
    assert O.shift_conv(h, w)[:, 0].tolist() == [1.0, 12.0, 123.0, 234.0, 345.0]
    assert O.input_conv(h, w)[:, 0].tolist() == [2.0, 14.0, 126.0, 238.0, 350.0]
    # rotation: position 0 leaves the vector, a quarter turn swaps the pair; dimensions past `dims` pass
    v = torch.tensor([[[1.0, 0.0, 7.0, 9.0]]], dtype=F64).repeat(2, 1, 1)
    r = O.rotate_pairs(v, torch.tensor([0.0, math.pi / 2], dtype=F64), 2, 10000.0)
    assert torch.allclose(r[0], v[0]) and torch.allclose(r[1, 0], torch.tensor([0.0, 1.0, 7.0, 9.0], dtype=F64), atol=1e-12)
    # temperature steps where (p + 1) / every crosses an integer
    t = O.query_temperature(torch.tensor([0, 5, 6, 12, 13]), 0.5, 7)
    assert torch.allclose(t, 1 + 0.5 * torch.log(torch.tensor([1.0, 1.0, 2.0, 2.0, 3.0], dtype=F64)))
    # a sink of weight e^s beside one key of score 0: the value is scaled by 1 / (1 + e^s)
    o = O.causal_softmax_attention(torch.zeros(1, 1, 2, dtype=F64), torch.zeros(1, 1, 2, dtype=F64), torch.ones(1, 1, 3, dtype=F64), 1.0, 0.0,
                                   torch.tensor([math.log(3.0)]))
    assert torch.allclose(o, torch.full((1, 1, 3), 0.25, dtype=F64))
    # causal: the first row sees only itself
    q, k, vv = torch.randn(4, 2, 3, dtype=F64), torch.randn(4, 1, 3, dtype=F64), torch.randn(4, 1, 5, dtype=F64)
    assert torch.allclose(O.causal_softmax_attention(q, k, vv, 0.7)[0], vv[0].expand(2, 5))
    # the expert weight acts on the input: one expert, top 1, identity-like check through scaling
    W = {"m.router": torch.tensor([[0.0, 0.0]]), "m.e0.gate": torch.eye(2), "m.e0.up": torch.eye(2), "m.e0.down": torch.eye(2)}
    hh = torch.tensor([[2.0, -1.0]], dtype=F64)
    u = 0.5 * hh
    assert torch.allclose(O.moe(hh, W, "m.", {"router": {"experts": 1, "top": 1}}), O.silu(u) * u)


def test_oracle_recurrences_against_closed_forms():
    # selective scan with constant inputs: S_t = sum_{s<=t} decay^(t-s) dt x B
    p, inner, N, T = "r.", 2, 3, 6
    W = {p + "in": torch.cat([torch.eye(2), torch.eye(2)]), p + "conv": torch.tensor([[0.0, 1.0], [0.0, 1.0]]), p + "conv.b": torch.zeros(2),
         p + "x": torch.zeros(1 + 2 * N, 2), p + "dt": torch.zeros(2, 1), p + "dt.b": torch.tensor([0.3, -0.2]), p + "A_log": torch.zeros(2, N),
         p + "D": torch.tensor([0.5, 0.25]), p + "o": torch.eye(2)}
    h = torch.tensor([[1.0, 2.0]], dtype=F64).repeat(T, 1)
    y = O.selective_scan(h, W, p, {"inner": inner, "state": N, "dt_rank": 1, "conv": 2})
    x = O.silu(h)
    assert torch.allclose(y, (torch.tensor([0.5, 0.25], dtype=F64) * x) * O.silu(h))      # B = C = 0: only the skip path D x, gated
    # gated linear attention: with alpha = 1 (a huge bias) and q = k the read-out is the running sum of (q . k_s) v_s
    H, d, dv = 1, 2, 2
    W = {"g.q": torch.eye(2), "g.k": torch.eye(2), "g.v": torch.eye(2), "g.g": torch.eye(2), "g.a1": torch.zeros(1, 2), "g.a2": torch.zeros(2, 1),
         "g.a2.b": torch.full((2,), 80.0), "g.norm": torch.ones(2), "g.o": torch.eye(2)}
    hh = torch.tensor([[1.0, 0.0], [0.0, 2.0], [1.0, 1.0]], dtype=F64)
    out = O.gla_mixer(hh, W, "g.", {"heads": H, "dim": d, "vdim": dv, "tau": 4.0}, 0.0)
    S = torch.zeros(2, 2, dtype=F64)
    for t in range(3):
        S = S + hh[t][:, None] * hh[t][None, :]
        o = (S.T @ hh[t]) * d ** -0.5
        want = o / o.pow(2).mean().sqrt() * O.silu(hh[t])
        assert torch.allclose(out[t], want)
