"""A toy architecture that the package has never seen, taken the way a user would add one.

Importing this module registers, from outside ``tesseract_b200``:

* ``toy_running_mean``: a mixer whose paged cache is not keys and values but one small latent vector per token
  (its cache need gives its own page shape), read back through the block table;
* ``toy_state_decay``: a mixer with fixed-size state per request (no pages at all);
* ``toy_top1_experts``: a feed-forward that routes every row to one of its experts;
* the architecture ``ToyMixedForTests``: a typed reader of its own ``config.json`` keys and a builder of the
  model description (an attention layer of the package, then the two toy mixers), with tied embeddings.

Nothing here is a model of anyone's: the parts are written with plain torch operations and exist to show that
registering, loading, generating and replaying need no change under ``tesseract_b200/``.  ``plain_forward`` is the
whole-sequence float64 answer the tests compare with.  The command line and the replay program learn of this
module through ``--plugin tests.toy_architecture``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

import torch

from tesseract_b200.config import (Architecture, ConfigError, LayerSpec, ModelSpec, PartSpec, RunEntry,
                                   register_architecture, require)
from tesseract_b200.parts import FEED_FORWARDS, MIXERS, FeedForward, Mixer, PagedNeed, StateNeed
from tesseract_b200.weights.loader import ExpectedTensor

ARCHITECTURE = "ToyMixedForTests"


# ----------------------------------------------------------------------------- parts


@dataclass(frozen=True)
class LatentNeed(PagedNeed):
    """One float32 vector of ``width`` numbers per token: a page is ``[page_size, width]``."""

    width: int = 0
    window: Optional[int] = None
    dtype: Optional[torch.dtype] = torch.float32

    def page_shape(self, page_size: int) -> Tuple[int, ...]:
        return (page_size, self.width)


if "toy_running_mean" not in MIXERS.kinds():

    @MIXERS.register("toy_running_mean")
    class ToyRunningMean(Mixer):
        """``out[t] = mean_{s <= t}(x[s] Wl^T) Wo^T``: every token's latent goes into the request's pages, every row
        reads all latents up to its own position back through the block table."""

        def __init__(self, spec, tensors, runtime):
            super().__init__(spec, tensors, runtime)
            self.width = int(spec.params["latent"])
            self.down = tensors["down"].to(device=runtime.device, dtype=torch.float32)
            self.up = tensors["up"].to(device=runtime.device, dtype=torch.float32)

        @classmethod
        def expected_tensors(cls, spec):
            hidden, width = int(spec.params["hidden_size"]), int(spec.params["latent"])
            return {spec.weights["down"]: ExpectedTensor((width, hidden)),
                    spec.weights["up"]: ExpectedTensor((hidden, width))}

        @classmethod
        def random_tensor(cls, spec, role, shape, generator):
            return torch.randn(shape, generator=generator) * 0.3

        def cache_need(self):
            return LatentNeed(width=self.width)

        def forward(self, x, ctx, cache):
            latent = x.float() @ self.down.T
            table = ctx.groups[cache.group].block_table
            size = cache.page_size
            out = torch.empty((x.shape[0], self.up.shape[0]), dtype=torch.float32, device=x.device)
            row = 0
            for seq, (begin, new) in enumerate(zip(ctx.host_begin, ctx.host_new)):
                every = torch.arange(begin + new, device=x.device)
                pages = table[seq, (every // size).long()].long()
                if cache.writes:
                    cache.storage[pages[begin:], every[begin:] % size] = latent[row:row + new]
                history = cache.storage[pages, every % size]                       # [begin + new, width]
                mean = history.cumsum(0)[begin:] / (every[begin:] + 1).to(torch.float32)[:, None]
                out[row:row + new] = mean @ self.up.T
                row += new
            return out.to(x.dtype)

    @MIXERS.register("toy_state_decay")
    class ToyStateDecay(Mixer):
        """``state = decay * state + x * w`` per request; the output is the state."""

        def __init__(self, spec, tensors, runtime):
            super().__init__(spec, tensors, runtime)
            self.size, self.decay = int(spec.params["hidden_size"]), float(spec.params["decay"])
            self.w = runtime.vector_f32(tensors["w"])

        @classmethod
        def expected_tensors(cls, spec):
            return {spec.weights["w"]: ExpectedTensor((int(spec.params["hidden_size"]),))}

        @classmethod
        def random_tensor(cls, spec, role, shape, generator):
            return 1.0 + 0.1 * torch.randn(shape, generator=generator)

        def cache_need(self):
            return StateNeed((self.size,), torch.float32)

        def forward(self, x, ctx, cache):
            out = torch.empty_like(x)
            row = 0
            for slot, new in zip(ctx.host_slots, ctx.host_new):
                state = cache.storage[slot]
                for _ in range(new):
                    state.mul_(self.decay).add_(x[row].float() * self.w)
                    out[row] = state.to(x.dtype)
                    row += 1
            return out

    @FEED_FORWARDS.register("toy_top1_experts")
    class ToyTop1Experts(FeedForward):
        """``y = relu(x W1[e]^T) W2[e]^T`` with ``e = argmax(x R^T)`` (router in 32-bit, lowest index on ties)."""

        def __init__(self, spec, tensors, runtime):
            super().__init__(spec, tensors, runtime)
            self.router, self.w1, self.w2 = (tensors[k].to(device=runtime.device, dtype=torch.float32)
                                             for k in ("router", "w1", "w2"))

        @classmethod
        def expected_tensors(cls, spec):
            p, w = spec.params, spec.weights
            e, h, i = int(p["experts"]), int(p["hidden_size"]), int(p["intermediate_size"])
            return {w["router"]: ExpectedTensor((e, h)), w["w1"]: ExpectedTensor((e, i, h)),
                    w["w2"]: ExpectedTensor((e, h, i))}

        @classmethod
        def random_tensor(cls, spec, role, shape, generator):
            return torch.randn(shape, generator=generator) * (1.0 if role == "router" else 0.2)

        def forward(self, x, ctx):
            rows = x.float()
            expert = (rows @ self.router.T).argmax(dim=1)
            hidden = torch.relu(torch.einsum("th,tih->ti", rows, self.w1[expert]))
            return torch.einsum("ti,thi->th", hidden, self.w2[expert]).to(x.dtype)


# ----------------------------------------------------------------------------- configuration and description


@dataclass(frozen=True)
class ToyConfig:
    width: int
    vocabulary: int
    heads: int
    head_width: int
    inner: int
    latent: int
    experts: int
    decay: float
    epsilon: float
    positions: int
    stop_token: int

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "ToyConfig":
        cfg = cls(width=require(data, "width", int), vocabulary=require(data, "vocabulary", int),
                  heads=require(data, "heads", int), head_width=require(data, "head_width", int),
                  inner=require(data, "inner", int), latent=require(data, "latent", int),
                  experts=require(data, "experts", int), decay=float(require(data, "decay", (int, float))),
                  epsilon=float(require(data, "epsilon", (int, float))), positions=require(data, "positions", int),
                  stop_token=require(data, "stop_token", int))
        if not 0 <= cfg.stop_token < cfg.vocabulary:
            raise ConfigError("stop_token must lie inside the vocabulary")
        return cfg


def toy_spec(cfg: ToyConfig) -> ModelSpec:
    def norm(name):
        return PartSpec.make("rms_norm", {"size": cfg.width, "eps": cfg.epsilon}, {"weight": name})

    def swiglu(i):
        return PartSpec.make("swiglu", {"hidden_size": cfg.width, "intermediate_size": cfg.inner},
                             {"gate": f"blocks.{i}.gate", "up": f"blocks.{i}.up", "down": f"blocks.{i}.down"})

    mixers = [
        PartSpec.make("attention", {"hidden_size": cfg.width, "num_heads": cfg.heads, "num_kv_heads": 1,
                                    "head_dim": cfg.head_width, "window": None, "scale": None},
                      {r: f"blocks.0.{r}" for r in "qkvo"},
                      {"position": PartSpec.make("rotary", {"head_dim": cfg.head_width, "theta": 100.0, "scaling": None})}),
        PartSpec.make("toy_running_mean", {"hidden_size": cfg.width, "latent": cfg.latent},
                      {"down": "blocks.1.latent_down", "up": "blocks.1.latent_up"}),
        PartSpec.make("toy_state_decay", {"hidden_size": cfg.width, "decay": cfg.decay}, {"w": "blocks.2.w"}),
    ]
    feed_forwards = [swiglu(0), swiglu(1),
                     PartSpec.make("toy_top1_experts", {"experts": cfg.experts, "hidden_size": cfg.width,
                                                        "intermediate_size": cfg.inner},
                                   {"router": "blocks.2.router", "w1": "blocks.2.w1", "w2": "blocks.2.w2"})]
    layers = tuple(LayerSpec.make("pre_norm", mixers[i], feed_forwards[i],
                                  {"input": norm(f"blocks.{i}.norm1"), "post_mixer": norm(f"blocks.{i}.norm2")})
                   for i in range(3))
    sizes = {"vocab_size": cfg.vocabulary, "hidden_size": cfg.width}
    return ModelSpec(architecture=ARCHITECTURE, hidden_size=cfg.width, vocab_size=cfg.vocabulary,
                     max_positions=cfg.positions,
                     embedding=PartSpec.make("token_embedding", sizes, {"table": "tokens"}), layers=layers,
                     run_order=tuple(RunEntry(i) for i in range(3)), final_norm=norm("final_norm"),
                     head=PartSpec.make("lm_head", sizes, {"weight": "tokens"}),        # tied: the same tensor name
                     bos_token_id=0, eos_token_ids=(cfg.stop_token,))


register_architecture(Architecture(name=ARCHITECTURE, read_config=ToyConfig.from_dict, build_spec=toy_spec))

CONFIG = {"architectures": [ARCHITECTURE], "torch_dtype": "float32", "width": 40, "vocabulary": 97, "heads": 3,
          "head_width": 16, "inner": 56, "latent": 6, "experts": 3, "decay": 0.5, "epsilon": 1e-5, "positions": 256,
          "stop_token": 96}


# ----------------------------------------------------------------------------- the plain answer


def plain_forward(config: Mapping[str, Any], tensors: Mapping[str, torch.Tensor], tokens) -> torch.Tensor:
    """Logits ``[T, vocabulary]`` of a whole sequence in float64, no cache."""
    from tests.plain import llama

    cfg = ToyConfig.from_dict(config)
    w = {k: v.double() for k, v in tensors.items()}
    T = len(tokens)
    h = llama.embed(tokens, w["tokens"])
    for i in range(3):
        x = llama.rms_norm(h, w[f"blocks.{i}.norm1"], cfg.epsilon)
        if i == 0:
            d = cfg.head_width
            cos, sin = llama.rope_tables(range(T), llama.rope_inverse_frequencies(d, 100.0, None))
            q = llama.rotate_half((x @ w["blocks.0.q"].T).view(T, cfg.heads, d), cos, sin)
            k = llama.rotate_half((x @ w["blocks.0.k"].T).view(T, 1, d), cos, sin)
            v = (x @ w["blocks.0.v"].T).view(T, 1, d)
            mixed = llama.attention(q, k, v, d ** -0.5).reshape(T, cfg.heads * d) @ w["blocks.0.o"].T
        elif i == 1:
            latent = x @ w["blocks.1.latent_down"].T
            mean = latent.cumsum(0) / torch.arange(1, T + 1, dtype=torch.float64)[:, None]
            mixed = mean @ w["blocks.1.latent_up"].T
        else:
            state, rows = torch.zeros(cfg.width, dtype=torch.float64), []
            for t in range(T):
                state = cfg.decay * state + x[t] * w["blocks.2.w"]
                rows.append(state)
            mixed = torch.stack(rows)
        h = h + mixed
        m = llama.rms_norm(h, w[f"blocks.{i}.norm2"], cfg.epsilon)
        if i < 2:
            h = h + llama.swiglu(m, w[f"blocks.{i}.gate"], w[f"blocks.{i}.up"], w[f"blocks.{i}.down"])
        else:
            expert = (m @ w["blocks.2.router"].T).argmax(dim=1)
            hidden = torch.relu(torch.einsum("th,tih->ti", m, w["blocks.2.w1"][expert]))
            h = h + torch.einsum("ti,thi->th", hidden, w["blocks.2.w2"][expert])
    return llama.rms_norm(h, w["final_norm"], cfg.epsilon) @ w["tokens"].T
