"""CPU tests of the Tutizen host side: configuration reader, registry, and the oracle's own mechanisms (no GPU)."""
import math

import pytest
import torch

import tutizen_oracle as O


def _cfg():
    return {"architecture": "Tutizen", "vocab": 50, "width": 24, "norm": {"eps": 1e-4}, "residual_mult": 0.6, "layers": [
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 12, "scale": 0.3}, "mlp": {"kind": "dense", "ff": 40, "limit": 1.5}},
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 12, "scale": 0.2, "kv_from": 0},
         "mlp": {"kind": "moe", "expert": {"ff": 16, "limit": 1.0}, "shared": {"ff": 20, "limit": 2.5},
                 "router": {"experts": 8, "top": 2, "scale": 1.25, "groups": {"count": 4, "keep": 3}}}},
        {"type": "attention", "mixer": {"heads": 2, "kv_heads": 1, "dim": 16, "vdim": 8, "scale": 0.1}, "mlp": None}]}


def test_config_reader_takes_every_size_and_constant_from_the_config():
    from sglang.srt.models.tutizen import TutizenConfig
    from wf_bitnet import _lib
    c = TutizenConfig.from_dict(_cfg())
    assert (c.vocab, c.width, c.eps, c.residual_mult) == (50, 24, 1e-4, 0.6)
    L = c.native_layers()
    assert [l.type for l in L] == [_lib.WF_SEQ_GQA_ATTENTION] * 3
    assert (L[0].heads, L[0].kv_heads, L[0].dim, L[0].vdim, L[0].kv_from) == (4, 2, 8, 12, -1)
    assert abs(L[0].scale - 0.3) < 1e-7 and abs(L[1].scale - 0.2) < 1e-7
    assert L[1].kv_from == 0 and L[2].kv_from == -1
    assert (L[0].has_ff, L[0].ff, L[0].ff_act) == (_lib.WF_SEQ_FF_DENSE, 40, _lib.WF_SEQ_ACT_CLAMPED) and abs(L[0].ff_limit - 1.5) < 1e-7
    assert (L[1].has_ff, L[1].experts, L[1].top, L[1].groups, L[1].keep, L[1].ff, L[1].shared_ff) == (_lib.WF_SEQ_FF_ROUTED, 8, 2, 4, 3, 16, 20)
    assert abs(L[1].router_scale - 1.25) < 1e-7 and abs(L[1].shared_limit - 2.5) < 1e-7 and (L[1].router_act, L[1].group_top, L[1].router_norm) == (1, 2, 1)
    assert L[2].has_ff == _lib.WF_SEQ_FF_NONE
    nc = _lib.SeqConfig()
    c.fill_native(nc)
    assert nc.block_form == _lib.WF_SEQ_BLOCK_POST and nc.pos_embed == 1 and abs(nc.residual_mult - 0.6) < 1e-7
    bad = _cfg()
    bad["layers"][0]["mixer"]["kv_from"] = 1
    with pytest.raises(ValueError):
        TutizenConfig.from_dict(bad).native_layers()
    bad = _cfg()
    bad["layers"][2]["type"] = "delta"
    with pytest.raises(ValueError):
        TutizenConfig.from_dict(bad).native_layers()


def test_registry_resolves_the_design():
    from wf_bitnet import registry
    assert registry.resolve({"architecture": "Tutizen"}).__name__ == "TutizenForCausalLM"
    assert registry.resolve({"architectures": ["TutizenForCausalLM"]}).__name__ == "TutizenForCausalLM"
    assert registry.resolve({"architecture": "Karusun"}).__name__ == "KarusunForCausalLM"


def test_oracle_is_causal_and_shares_the_cache():
    cfg = _cfg()
    w = {k: v.double() for k, v in O.random_weights(cfg, 5).items()}
    toks = [3, 14, 15, 9, 2, 6, 5, 35]
    full, taps = O.forward(toks, w, cfg)
    part, _ = O.forward(toks[:5], w, cfg)
    assert torch.allclose(full[:5], part, atol=1e-10)                     # later tokens change nothing earlier
    assert taps.shape == (3, 8, 24)
    # layer 1 reads layer 0's keys and values: changing layer 0's key projection moves layer 1's mixer output even with x held fixed
    x = torch.randn(6, 24, dtype=torch.float64)
    P0, P1 = O.sub(w, "l0.mix."), O.sub(w, "l1.mix.")
    kv = O.attention_keys_values(x, P0, cfg["layers"][0]["mixer"], 1e-4)
    kv2 = O.attention_keys_values(x, dict(P0, k=P0["k"] * 0.5 + 0.1), cfg["layers"][0]["mixer"], 1e-4)
    a = O.attention(x, P1, cfg["layers"][1]["mixer"], 1e-4, kv)[0]
    b = O.attention(x, P1, cfg["layers"][1]["mixer"], 1e-4, kv2)[0]
    assert (a - b).abs().max() > 1e-3
    # cached keys and values have unit root mean square per head
    assert torch.allclose((kv[0] ** 2).mean(-1), torch.ones(6, 2, dtype=torch.float64), atol=1e-3)
    assert torch.allclose((kv[1] ** 2).mean(-1), torch.ones(6, 2, dtype=torch.float64), atol=1e-3)


def test_oracle_router_and_units():
    z = torch.tensor([[3.0, -4.0, 2.0, 2.1, -9.0, -9.0, 1.9, 1.8]], dtype=torch.float64)
    ids, w = O.route(z, torch.zeros(8, dtype=torch.float64), 3, 4, 2, 1.5)
    assert sorted(ids[0].tolist()) == [2, 3, 6]                            # groups ranked by their two best, not by their best
    assert abs(float(w.sum()) - 1.5) < 1e-9
    g = torch.tensor([9.0]); u = torch.tensor([-9.0])
    assert abs(float(O.clamped_glu(g, u, 2.0)) - 2.0 * (1 / (1 + math.exp(-1.702 * 2.0))) * (-2.0 + 1.0)) < 1e-6
    x = torch.tensor([[3.0, 4.0]])
    assert torch.allclose(O.scalar_rms_norm(x, 2.0, 0.0), x / math.sqrt(12.5) * 2.0)
