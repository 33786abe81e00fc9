"""Tutizen: a decoder-only stack of attention layers.  The embedding gets a sinusoidal position vector; every sublayer reads the residual
stream itself and its OUTPUT is RMS-normalised with one gain, multiplied by a constant and added.  The mixer is grouped-query softmax
attention without rotation: queries, keys and values divided by their root mean square per head, a linear distance penalty per head
(slope 2^(-8 (h + 1) / heads)), a per-head sigmoid output gate, biases on the projections, and optionally the cached keys and values of an
earlier layer instead of projections of its own.  The feed-forward is a clamped gated unit (g * sigmoid(1.702 g) * (u + 1)), dense or
routed: sigmoid router, additive choice correction, groups ranked by the sum of their two best choice scores, weights normalised over the
chosen experts and scaled, plus a shared expert behind a sigmoid gate.

This module is the model's configuration reader and its binding to the native engine (libwf_seq.so); it computes nothing itself.
config.json keys read here: architecture, vocab, width, residual_mult, norm.eps, layers[].{type, mixer.{heads, kv_heads, dim, vdim, scale,
kv_from}, mlp.{kind, ff, limit, expert.{ff, limit}, router.{experts, top, scale, groups.{count, keep}}, shared.{ff, limit}}}.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List

from wf_bitnet import _lib
from wf_bitnet._lib import SeqConfig, SeqLayer
from wf_bitnet.seq_model import SeqCausalLM

NO_WINDOW = 1 << 30
# constants the design fixes
POSITION_BASE = 10000.0        # sinusoidal position vector
DISTANCE_EXPONENT = 8.0        # slope of head h: 2^(-8 (h + 1) / heads)
GROUP_TOP = 2                  # a group's score: the sum of its two largest choice scores


@dataclass
class TutizenConfig:
    vocab: int
    width: int
    eps: float
    residual_mult: float
    layers: List[dict] = field(default_factory=list)

    @staticmethod
    def from_dict(cfg: Dict) -> "TutizenConfig":
        out = TutizenConfig(vocab=int(cfg["vocab"]), width=int(cfg["width"]), eps=float(cfg["norm"]["eps"]),
                            residual_mult=float(cfg["residual_mult"]), layers=list(cfg["layers"]))
        if not out.layers:
            raise ValueError("config: 'layers' is empty")
        return out

    def fill_native(self, nc: SeqConfig) -> None:
        nc.block_form = _lib.WF_SEQ_BLOCK_POST
        nc.residual_mult = self.residual_mult
        nc.pos_embed, nc.pos_base = 1, POSITION_BASE

    def native_layers(self) -> List[SeqLayer]:
        res = []
        for i, L in enumerate(self.layers):
            if L["type"] != "attention":
                raise ValueError(f"config: layer {i} has unknown mixer type {L['type']!r}")
            m = L["mixer"]
            s = SeqLayer()
            s.type = _lib.WF_SEQ_GQA_ATTENTION
            s.heads, s.dim, s.vdim = int(m["heads"]), int(m["dim"]), int(m["vdim"])
            s.kv_heads = int(m.get("kv_heads", s.heads))
            s.scale = float(m["scale"])
            s.window = NO_WINDOW
            s.qk_norm = s.v_norm = s.proj_bias = s.head_gate = 1
            s.dist_exp = DISTANCE_EXPONENT
            src = m.get("kv_from")
            s.kv_from = -1 if src is None else int(src)
            if s.kv_from >= i:
                raise ValueError(f"config: layer {i} takes keys and values from layer {s.kv_from}, which does not come before it")
            f = L.get("mlp")
            if f is None:
                s.has_ff = _lib.WF_SEQ_FF_NONE
            elif f["kind"] == "dense":
                s.has_ff, s.ff_act = _lib.WF_SEQ_FF_DENSE, _lib.WF_SEQ_ACT_CLAMPED
                s.ff, s.ff_limit = int(f["ff"]), float(f["limit"])
            elif f["kind"] == "moe":
                r = f["router"]
                s.has_ff, s.ff_act = _lib.WF_SEQ_FF_ROUTED, _lib.WF_SEQ_ACT_CLAMPED
                s.experts, s.identity, s.top = int(r["experts"]), 0, int(r["top"])
                g = r.get("groups") or {}
                s.groups = int(g.get("count", 1))
                s.keep = int(g.get("keep", s.groups))
                s.ff, s.ff_limit = int(f["expert"]["ff"]), float(f["expert"]["limit"])
                s.router_act, s.group_top, s.router_norm = 1, GROUP_TOP, 1
                s.router_scale = float(r.get("scale", 1.0))
                sh = f.get("shared")
                if sh:
                    s.shared_ff, s.shared_limit = int(sh["ff"]), float(sh["limit"])
            else:
                raise ValueError(f"config: layer {i} has unknown feed-forward kind {f.get('kind')!r}")
            res.append(s)
        return res


class TutizenForCausalLM(SeqCausalLM):
    """Model class of the registry (weights, engine and step interface: wf_bitnet.seq_model.SeqCausalLM)."""

    architecture_names = ("Tutizen", "TutizenForCausalLM")

    @staticmethod
    def read_config(config: Dict) -> TutizenConfig:
        return TutizenConfig.from_dict(config)


EntryClass = TutizenForCausalLM
