"""Karusun: a decoder-only stack whose layers each hold one mixer — sliding-window latent attention (a cached low-rank latent plus one
rotated key part shared by all heads, gated output) or a gated delta rule with short convolutions — followed by an optional routed
feed-forward (softmax router with a choice correction, group-limited top-k, identity experts).  Every sublayer is wrapped in grouped RMS
norms before and after, and reads its input through a short causal convolution whose tail is part of the sequence state.

This module is the model's configuration reader and its binding to the native engine (libwf_seq.so); it computes nothing itself.
config.json keys read here: architecture, vocab, width, norm.{eps,groups}, canon.taps, layers[].{type,mixer,mlp}.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np

from wf_bitnet import _lib, checkpoint
from wf_bitnet._lib import SeqConfig, SeqLayer
from wf_bitnet.seq_engine import SeqEngine

NO_WINDOW = 1 << 30


@dataclass
class KarusunConfig:
    vocab: int
    width: int
    eps: float
    norm_groups: int
    canon_taps: int
    layers: List[dict] = field(default_factory=list)
    has_canon: bool = True

    @staticmethod
    def from_dict(cfg: Dict) -> "KarusunConfig":
        norm = cfg.get("norm", {})
        out = KarusunConfig(vocab=int(cfg["vocab"]), width=int(cfg["width"]), eps=float(norm.get("eps", 1e-6)), norm_groups=int(norm.get("groups", 1)),
                            canon_taps=int((cfg.get("canon") or {}).get("taps", 1)), layers=list(cfg["layers"]), has_canon=bool(cfg.get("canon")))
        if not out.layers:
            raise ValueError("config: 'layers' is empty")
        return out

    def native_layers(self) -> List[SeqLayer]:
        res = []
        for i, L in enumerate(self.layers):
            m = L["mixer"]
            s = SeqLayer()
            s.heads, s.dim, s.vdim = int(m["heads"]), int(m["dim"]), int(m["vdim"])
            if L["type"] == "latent_attention":
                s.type = _lib.WF_SEQ_LATENT_ATTENTION
                s.rot_dim, s.kv_rank = int(m.get("rot_dim", 0)), int(m["kv_rank"])
                s.window = int(m["mask"]["size"]) if m.get("mask") else NO_WINDOW
                rot = m.get("rot") or {}
                s.rope_dims = int(rot.get("dims", s.rot_dim))
                s.rope_base = float(rot.get("base", 10000.0))
                s.scale = float(m["scale"]) if "scale" in m else float((s.dim + s.rot_dim) ** -0.5)
            elif L["type"] == "delta":
                s.type = _lib.WF_SEQ_DELTA
                s.kv_heads, s.conv = int(m.get("kv_heads", s.heads)), int(m.get("conv", 1))
            else:
                raise ValueError(f"config: layer {i} has unknown mixer type {L['type']!r}")
            f = L.get("mlp")
            if f is not None:
                if f.get("kind", "moe") != "moe":
                    raise ValueError(f"config: layer {i} has unknown feed-forward kind {f.get('kind')!r}")
                r = f["router"]
                s.has_ff = 1
                s.experts, s.identity, s.top = int(r["experts"]), int(r.get("identity", 0)), int(r["top"])
                g = r.get("groups") or {}
                s.groups, s.keep = int(g.get("count", 1)), int(g.get("keep", g.get("count", 1)))
                s.ff = int(f.get("expert", {}).get("ff", 0))
            res.append(s)
        return res


class KarusunForCausalLM:
    """Model class of the registry: owns a native engine sized for `max_tokens` cached tokens and `slots` live sequences."""

    architecture_names = ("Karusun", "KarusunForCausalLM")
    min_page_size = 1

    def __init__(self, config: Dict, *, dtype: str = "bfloat16", max_tokens: int = 4096, slots: int = 4, page_size: int = 16,
                 max_step_tokens: int = 1024, build: bool = False):
        if dtype not in ("bfloat16", "float32"):
            raise ValueError(f"dtype must be bfloat16 or float32, got {dtype!r}")
        self.config = KarusunConfig.from_dict(config)
        c = self.config
        self.dtype = dtype
        self.page_size = page_size
        pages = max(1, (max_tokens + page_size - 1) // page_size)
        self.native_config = SeqConfig(_lib.WF_SEQ_F32 if dtype == "float32" else _lib.WF_SEQ_BF16, c.vocab, c.width, len(c.layers), c.eps,
                                       c.norm_groups, c.canon_taps, page_size, pages, slots, max_step_tokens)
        self.engine = SeqEngine(self.native_config, c.native_layers(), build=build)
        self.vocab = c.vocab
        self.max_step_tokens = max_step_tokens

    @classmethod
    def from_pretrained(cls, model_dir, config=None, **serving):
        """Model folder (config.json + model.safetensors) -> a loaded model; `serving`: dtype, max_tokens, slots, page_size,
        max_step_tokens, build."""
        from pathlib import Path
        cfg = config if config is not None else checkpoint.read_config(model_dir)
        m = cls(cfg, **serving)
        m.load_safetensors(Path(model_dir) / "model.safetensors")
        return m

    # ---- weights
    def load_weights(self, weights: Iterable[Tuple[str, np.ndarray, str]]) -> None:
        """weights: (checkpoint name, array, safetensors dtype string) — bfloat16 as uint16 bit patterns (wf_bitnet.checkpoint)."""
        wanted = {n for n, _, _ in self.engine.expected_tensors()}
        for name, a, dt in weights:
            if name not in wanted:
                continue
            self.engine.set_tensor(name, checkpoint.to_float32(a, dt) if self.dtype == "float32" else checkpoint.to_bfloat16_bits(a, dt))
        # tensors of parts the configuration does not mention are neutral: no input convolution (zero taps), no choice correction
        for n, count, loaded in self.engine.expected_tensors():
            if not loaded and ((not self.config.has_canon and n.endswith((".canon1", ".canon2"))) or n.endswith(".mlp.correction")):
                self.engine.set_tensor(n, np.zeros(count, dtype=np.float32 if self.dtype == "float32" else np.uint16))
        missing = [n for n, _, loaded in self.engine.expected_tensors() if not loaded]
        if missing:
            raise KeyError(f"checkpoint lacks {len(missing)} tensors, first: {missing[:4]}")
        self.engine.finalize()

    def load_safetensors(self, path) -> None:
        f = checkpoint.SafetensorsFile(path)
        try:
            self.load_weights(f.items())
        finally:
            f.close()

    # ---- the step interface the scheduler and the trace replay drive
    def admit(self) -> int:
        return self.engine.admit()

    def release(self, slot: int) -> None:
        self.engine.release(slot)

    def free_pages(self) -> int:
        return self.engine.free_pages()

    def free_slots(self) -> int:
        return self.engine.free_slots()

    def pages_for(self, tokens: int) -> int:
        return (tokens + self.page_size - 1) // self.page_size

    def step(self, slots: Sequence[int], counts: Sequence[int], tokens: Sequence[int], want: Sequence[int] = (), fetch: bool = True):
        return self.engine.step(slots, counts, tokens, want, fetch)

    def sample(self, nrows: int, temperature: float = 0.0, top_k: int = 0, top_p: float = 1.0, uniforms=None) -> np.ndarray:
        return self.engine.sample(nrows, temperature, top_k, top_p, uniforms)

    def close(self) -> None:
        self.engine.close()


EntryClass = KarusunForCausalLM
