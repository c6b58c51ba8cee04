"""Each part of a decoder alone, and a toy mixer with state of its own that the framework has never seen."""

import math

import numpy as np
import pytest
import torch

from tests.plain import llama

pytestmark = pytest.mark.gpu


def runtime(dtype):
    from tesseract_b200.parts import Runtime

    return Runtime(dtype, torch.device("cuda", 0))


def context_for(cache, requests, news):
    """A StepContext for the given live requests bringing ``news[i]`` tokens each (pages already extended)."""
    from tesseract_b200.parts import GroupView, StepContext

    begins = [cache.length(r) for r in requests]
    slots = [cache.slot(r) for r in requests]
    positions = [p for b, n in zip(begins, news) for p in range(b, b + n)]
    seq_of_row = [s for s, n in enumerate(news) for _ in range(n)]
    columns = -(-max(b + n for b, n in zip(begins, news)) // cache.page_size)
    groups = []
    for index, g in enumerate(cache.groups):
        table = None
        if g.pool is not None:
            table = torch.from_numpy(cache.block_table_rows(index, slots, columns)).cuda()
        groups.append(GroupView(table, cache.page_size if g.pool is not None else 0))
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    return StepContext(num_rows=len(positions), num_seqs=len(requests), token_ids=i32([0] * len(positions)),
                       positions=i32(positions), seq_of_row=i32(seq_of_row),
                       row_start=i32(np.concatenate([[0], np.cumsum(news)]).tolist()), seq_begin=i32(begins),
                       state_slots=i32(slots), groups=groups, host_new=news, host_begin=begins, host_slots=slots,
                       max_new=max(news), max_context=max(b + n for b, n in zip(begins, news)))


@pytest.mark.parametrize("dtype, tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
def test_norm_feed_forward_embedding_head(dtype, tol):
    from tesseract_b200.config import PartSpec
    from tesseract_b200.parts import EMBEDDINGS, FEED_FORWARDS, HEADS, NORMS

    torch.manual_seed(0)
    rt = runtime(dtype)
    hidden, inter, vocab, rows = 40, 72, 57, 9
    x = torch.randn(rows, hidden).to(dtype)
    w = (1 + 0.1 * torch.randn(hidden)).to(dtype)
    norm = NORMS.get("rms_norm")(PartSpec.make("rms_norm", {"size": hidden, "eps": 1e-4}, {"weight": "n"}),
                                 {"weight": w}, rt)
    got = norm.forward(x.cuda()).cpu().double()
    torch.testing.assert_close(got, llama.rms_norm(x.double(), w.double(), 1e-4), rtol=tol, atol=tol)

    gate, up, down = (torch.randn(inter, hidden) * 0.2).to(dtype), (torch.randn(inter, hidden) * 0.2).to(dtype), \
        (torch.randn(hidden, inter) * 0.2).to(dtype)
    spec = PartSpec.make("swiglu", {"hidden_size": hidden, "intermediate_size": inter},
                         {"gate": "g", "up": "u", "down": "d"})
    ffn = FEED_FORWARDS.get("swiglu")(spec, {"gate": gate, "up": up, "down": down}, rt)
    assert set(ffn.expected_tensors(spec)) == {"g", "u", "d"}
    got = ffn.forward(x.cuda(), None).cpu().double()
    torch.testing.assert_close(got, llama.swiglu(x.double(), gate.double(), up.double(), down.double()),
                               rtol=tol, atol=tol)

    table = torch.randn(vocab, hidden).to(dtype)
    sizes = {"vocab_size": vocab, "hidden_size": hidden}
    emb = EMBEDDINGS.get("token_embedding")(PartSpec.make("token_embedding", sizes, {"table": "e"}), {"table": table}, rt)
    tokens = torch.tensor([0, 56, 3, 3], dtype=torch.int32, device="cuda")
    assert torch.equal(emb.forward(tokens).cpu(), table[tokens.cpu().long()])
    head = HEADS.get("lm_head")(PartSpec.make("lm_head", sizes, {"weight": "e"}), {"weight": table}, rt)
    logits = head.forward(x.cuda())
    assert logits.dtype == torch.float32
    torch.testing.assert_close(logits.cpu().double(), x.double() @ table.double().T, rtol=tol, atol=tol * 5)


@pytest.mark.parametrize("dtype, tol", [(torch.float32, 2e-5), (torch.bfloat16, 3e-2)])
@pytest.mark.parametrize("window", [None, 20])
def test_attention_part_alone_in_portions(dtype, tol, window):
    """The attention mixer with its own cache, fed a sequence in three portions beside a second request."""
    from tesseract_b200.cache import CacheManager
    from tesseract_b200.config import PartSpec
    from tesseract_b200.parts import MIXERS

    torch.manual_seed(1)
    rt = runtime(dtype)
    hidden, nh, nkv, d = 40, 6, 2, 16
    position = PartSpec.make("rotary", {"head_dim": d, "theta": 1000.0, "scaling": None})
    spec = PartSpec.make("attention", {"hidden_size": hidden, "num_heads": nh, "num_kv_heads": nkv, "head_dim": d,
                                       "window": window, "scale": 0.2},
                         {"q": "q", "k": "k", "v": "v", "o": "o"}, {"position": position})
    weights = {"q": torch.randn(nh * d, hidden) * 0.2, "k": torch.randn(nkv * d, hidden) * 0.2,
               "v": torch.randn(nkv * d, hidden) * 0.2, "o": torch.randn(hidden, nh * d) * 0.2}
    weights = {k: v.to(dtype) for k, v in weights.items()}
    mixer = MIXERS.get("attention")(spec, weights, rt)
    need = mixer.cache_need()
    assert (need.num_kv_heads, need.head_dim, need.window) == (nkv, d, window)
    cache = CacheManager([need], [None], num_pages=16, page_size=16, max_requests=2, dtype=dtype, device=rt.device,
                         max_step_tokens=64)
    xs = {"a": torch.randn(70, hidden).to(dtype), "b": torch.randn(45, hidden).to(dtype)}
    cuts = {"a": [33, 2, 35], "b": [1, 43, 1]}
    outs = {"a": [], "b": []}
    for r in xs:
        assert cache.admit(r)
    for step in range(3):
        news = [cuts[r][step] for r in ("a", "b")]
        for r, n in zip(("a", "b"), news):
            cache.extend(r, n)
        ctx = context_for(cache, ["a", "b"], news)
        x = torch.cat([xs[r][cache.length(r):cache.length(r) + n] for r, n in zip(("a", "b"), news)]).cuda()
        y = mixer.forward(x, ctx, cache.bindings[0]).cpu()
        at = 0
        for r, n in zip(("a", "b"), news):
            outs[r].append(y[at:at + n])
            at += n
            cache.commit(r, n)
    inv_freq = llama.rope_inverse_frequencies(d, 1000.0, None)
    w = {k: v.double() for k, v in weights.items()}
    for r, x in xs.items():
        T = x.shape[0]
        cos, sin = llama.rope_tables(range(T), inv_freq)
        q = llama.rotate_half((x.double() @ w["q"].T).view(T, nh, d), cos, sin)
        k = llama.rotate_half((x.double() @ w["k"].T).view(T, nkv, d), cos, sin)
        v = (x.double() @ w["v"].T).view(T, nkv, d)
        want = llama.attention(q, k, v, 0.2, window).reshape(T, nh * d) @ w["o"].T
        torch.testing.assert_close(torch.cat(outs[r]).double(), want, rtol=tol, atol=tol)
    cache.check()


# ----------------------------------------------------------------------------- a toy mixer with its own state


def register_toy_parts():
    from tesseract_b200.parts import MIXERS, Mixer, StateNeed
    from tesseract_b200.weights.loader import ExpectedTensor

    if "toy_decay" in MIXERS.kinds():
        return

    @MIXERS.register("toy_decay")
    class ToyDecay(Mixer):
        """s_t = decay * s_{t-1} + x_t * w ; y_t = s_t.  One vector of state per request, no pages."""

        def __init__(self, spec, tensors, runtime):
            super().__init__(spec, tensors, runtime)
            self.size = int(spec.params["size"])
            self.decay = float(spec.params["decay"])
            self.w = runtime.vector_f32(tensors["w"])

        @classmethod
        def expected_tensors(cls, spec):
            return {spec.weights["w"]: ExpectedTensor((int(spec.params["size"]),))}

        @classmethod
        def random_tensor(cls, spec, role, shape, generator):
            return 1.0 + 0.1 * torch.randn(shape, generator=generator)

        def cache_need(self):
            return StateNeed((self.size,), torch.float32)

        def forward(self, x, ctx, cache):
            out = torch.empty_like(x)
            row = 0
            for slot, new in zip(ctx.host_slots, ctx.host_new):      # rows of a request in order, state carried on
                state = cache.storage[slot]
                for _ in range(new):
                    state.mul_(self.decay).add_(x[row].float() * self.w)
                    out[row] = state.to(x.dtype)
                    row += 1
            return out


def toy_spec(layers=3, hidden=24, vocab=50):
    """attention, toy, attention reading layer 0's cache, then the toy layer once more (named twice)."""
    from tesseract_b200.config import LayerSpec, ModelSpec, PartSpec, RunEntry

    def norm(name):
        return PartSpec.make("rms_norm", {"size": hidden, "eps": 1e-5}, {"weight": name})

    def ffn(i):
        return PartSpec.make("swiglu", {"hidden_size": hidden, "intermediate_size": 32},
                             {"gate": f"l{i}.g", "up": f"l{i}.u", "down": f"l{i}.d"})

    def attn(i):
        return PartSpec.make("attention", {"hidden_size": hidden, "num_heads": 3, "num_kv_heads": 1, "head_dim": 16,
                                           "window": None, "scale": None},
                             {"q": f"l{i}.q", "k": f"l{i}.k", "v": f"l{i}.v", "o": f"l{i}.o"},
                             {"position": PartSpec.make("rotary", {"head_dim": 16, "theta": 100.0, "scaling": None})})

    toy = PartSpec.make("toy_decay", {"size": hidden, "decay": 0.5}, {"w": "l1.w"})
    mixers = [attn(0), toy, attn(2)]
    specs = [LayerSpec.make("pre_norm", mixers[i], ffn(i), {"input": norm(f"l{i}.n1"), "post_mixer": norm(f"l{i}.n2")})
             for i in range(layers)]
    sizes = {"vocab_size": vocab, "hidden_size": hidden}
    return ModelSpec(architecture="ToyForTests", hidden_size=hidden, vocab_size=vocab, max_positions=256,
                     embedding=PartSpec.make("token_embedding", sizes, {"table": "emb"}), layers=tuple(specs),
                     run_order=(RunEntry(0), RunEntry(1), RunEntry(2, cache_of=0), RunEntry(1)),
                     final_norm=norm("fn"), head=PartSpec.make("lm_head", sizes, {"weight": "head"}))


def toy_plain(tensors, tokens, hidden=24):
    """Whole sequence, float64, no cache."""
    w = {k: v.double() for k, v in tensors.items()}
    T = len(tokens)
    cos, sin = llama.rope_tables(range(T), llama.rope_inverse_frequencies(16, 100.0, None))
    h = llama.embed(tokens, w["emb"])
    kv0 = None
    for layer in (0, 1, 2, 1):
        x = llama.rms_norm(h, w[f"l{layer}.n1"], 1e-5)
        if layer == 1:
            state, rows = torch.zeros(hidden, dtype=torch.float64), []
            for t in range(T):
                state = 0.5 * state + x[t] * w["l1.w"]
                rows.append(state)
            mixed = torch.stack(rows)
        else:
            q = llama.rotate_half((x @ w[f"l{layer}.q"].T).view(T, 3, 16), cos, sin)
            if layer == 0:
                kv0 = (llama.rotate_half((x @ w["l0.k"].T).view(T, 1, 16), cos, sin), (x @ w["l0.v"].T).view(T, 1, 16))
            mixed = llama.attention(q, kv0[0], kv0[1], 0.25).reshape(T, 48) @ w[f"l{layer}.o"].T
        h = h + mixed
        m = llama.rms_norm(h, w[f"l{layer}.n2"], 1e-5)
        h = h + llama.swiglu(m, w[f"l{layer}.g"], w[f"l{layer}.u"], w[f"l{layer}.d"])
    return llama.rms_norm(h, w["fn"], 1e-5) @ w["head"].T


def test_toy_mixer_with_state_registers_builds_and_steps():
    """A new mixer kind with fixed-size state, a layer named twice, and a layer reading another's cache."""
    from tesseract_b200.engine import StepEntry, make_stepper
    from tesseract_b200.models import DecoderModel, expected_tensors, tensor_roles

    register_toy_parts()
    spec = toy_spec()
    g = torch.Generator().manual_seed(0)
    tensors = {name: cls.random_tensor(part, role, tuple(want.shape), g) * (5 if role in "qkvo" else 1)
               for cls, part, role, name, want in tensor_roles(spec)}
    assert set(tensors) == set(expected_tensors(spec)) and "l1.w" in tensors
    model = DecoderModel(spec, tensors, runtime(torch.float32))
    needs = model.cache_needs()
    # entry 2 keeps no cache (it reads entry 0's); the toy layer's two runs each keep their own state
    assert needs[2] is None and type(needs[1]).__name__ == "StateNeed" and needs[3] == needs[1]
    stepper = make_stepper(model, capacity_tokens=256, max_requests=3)
    assert len(stepper.cache.groups) == 2 and stepper.cache.groups[1].storage.shape[:2] == (2, 3 + 1)
    rng = np.random.default_rng(0)
    seqs = {"p": rng.integers(0, 50, 37).tolist(), "q": rng.integers(0, 50, 20).tolist()}
    plain = {r: toy_plain(tensors, t) for r, t in seqs.items()}
    cuts = {"p": [5, 1, 20, 2, 9], "q": [20]}
    got = {r: [] for r in seqs}
    for r in seqs:
        assert stepper.cache.admit(r)
    at = {"p": 0, "q": 0}
    for step in range(5):
        entries = []
        for r in ("p", "q"):
            if step < len(cuts[r]):
                n = cuts[r][step]
                entries.append(StepEntry(r, seqs[r][at[r]:at[r] + n], list(range(n))))
                at[r] += n
        logits = stepper.step(entries).cpu().double()
        k = 0
        for e in entries:
            got[e.request].append(logits[k:k + len(e.tokens)])
            k += len(e.tokens)
    for r in seqs:
        torch.testing.assert_close(torch.cat(got[r]), plain[r], rtol=2e-5, atol=2e-5)
    # a slot that is used again starts from empty state
    stepper.cache.release("q")
    assert stepper.cache.admit("q2")
    again = stepper.step([StepEntry("q2", seqs["q"], [19])]).cpu().double()
    torch.testing.assert_close(again[0], plain["q"][19], rtol=2e-5, atol=2e-5)


def register_toy_routing_and_position():
    """A feed-forward that routes each row to one of its experts, and a position encoding that rotates adjacent
    pairs: two more kinds that the framework has never seen (written with torch operations; they are toys)."""
    from tesseract_b200.parts import FEED_FORWARDS, POSITION_ENCODINGS, FeedForward, PositionEncoding
    from tesseract_b200.weights.loader import ExpectedTensor

    if "toy_top1" in FEED_FORWARDS.kinds():
        return

    @FEED_FORWARDS.register("toy_top1")
    class ToyTop1(FeedForward):
        """y = relu(x W1[e]^T) W2[e]^T with e = argmax(x R^T) (router logits in 32-bit, lowest index on ties)."""

        def __init__(self, spec, tensors, runtime):
            super().__init__(spec, tensors, runtime)
            self.router = tensors["router"].to(device=runtime.device, dtype=torch.float32)
            self.w1 = tensors["w1"].to(device=runtime.device, dtype=torch.float32)
            self.w2 = tensors["w2"].to(device=runtime.device, dtype=torch.float32)

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

    @POSITION_ENCODINGS.register("toy_adjacent_pairs")
    class ToyAdjacentPairs(PositionEncoding):
        """(x[2i], x[2i+1]) rotated by position * theta^(-2i/d): no inverse-frequency table for the kernels, so the
        mixer calls ``apply`` on its query and key views."""

        def __init__(self, spec, tensors, runtime):
            super().__init__(spec, tensors, runtime)
            d = int(spec.params["head_dim"])
            self.freq = torch.tensor([float(spec.params["theta"]) ** (-2.0 * i / d) for i in range(d // 2)],
                                     dtype=torch.float32, device=runtime.device)

        def apply(self, q, k, positions):
            angle = positions.to(torch.float32)[:, None] * self.freq[None, :]
            cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
            for x in (q, k):
                even, odd = x[..., 0::2].float(), x[..., 1::2].float()
                new_even, new_odd = even * cos - odd * sin, odd * cos + even * sin   # both before either is stored
                x[..., 0::2] = new_even.to(x.dtype)
                x[..., 1::2] = new_odd.to(x.dtype)


def test_toy_routed_feed_forward_and_position_encoding_build_and_step():
    from tesseract_b200.config import LayerSpec, ModelSpec, PartSpec, RunEntry
    from tesseract_b200.engine import StepEntry, make_stepper
    from tesseract_b200.models import DecoderModel, tensor_roles

    register_toy_routing_and_position()
    hidden, vocab, d = 32, 47, 16

    def norm(name):
        return PartSpec.make("rms_norm", {"size": hidden, "eps": 1e-5}, {"weight": name})

    def layer(i):
        mixer = PartSpec.make("attention", {"hidden_size": hidden, "num_heads": 2, "num_kv_heads": 1, "head_dim": d,
                                            "window": None, "scale": None},
                              {"q": f"l{i}.q", "k": f"l{i}.k", "v": f"l{i}.v", "o": f"l{i}.o"},
                              {"position": PartSpec.make("toy_adjacent_pairs", {"head_dim": d, "theta": 50.0})})
        ffn = PartSpec.make("toy_top1", {"experts": 3, "hidden_size": hidden, "intermediate_size": 24},
                            {"router": f"l{i}.r", "w1": f"l{i}.w1", "w2": f"l{i}.w2"})
        return LayerSpec.make("pre_norm", mixer, ffn, {"input": norm(f"l{i}.n1"), "post_mixer": norm(f"l{i}.n2")})

    sizes = {"vocab_size": vocab, "hidden_size": hidden}
    spec = ModelSpec(architecture="RoutedForTests", hidden_size=hidden, vocab_size=vocab, max_positions=128,
                     embedding=PartSpec.make("token_embedding", sizes, {"table": "emb"}),
                     layers=(layer(0), layer(1)), run_order=(RunEntry(0), RunEntry(1)),
                     final_norm=norm("fn"), head=PartSpec.make("lm_head", sizes, {"weight": "head"}))
    g = torch.Generator().manual_seed(11)
    tensors = {name: cls.random_tensor(part, role, tuple(want.shape), g) * (4 if role in "qk" else 1)
               for cls, part, role, name, want in tensor_roles(spec)}
    model = DecoderModel(spec, tensors, runtime(torch.float32))
    stepper = make_stepper(model, capacity_tokens=128, max_requests=2)

    def plain(tokens):
        w = {k: v.double() for k, v in tensors.items()}
        T = len(tokens)
        freq = torch.tensor([50.0 ** (-2.0 * i / d) for i in range(d // 2)], dtype=torch.float32)
        angle = (torch.arange(T, dtype=torch.float32)[:, None] * freq[None, :]).double()
        cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]

        def rotate(x):
            out = torch.empty_like(x)
            out[..., 0::2] = x[..., 0::2] * cos - x[..., 1::2] * sin
            out[..., 1::2] = x[..., 1::2] * cos + x[..., 0::2] * sin
            return out

        h = llama.embed(tokens, w["emb"])
        for i in range(2):
            x = llama.rms_norm(h, w[f"l{i}.n1"], 1e-5)
            q, k = rotate((x @ w[f"l{i}.q"].T).view(T, 2, d)), rotate((x @ w[f"l{i}.k"].T).view(T, 1, d))
            v = (x @ w[f"l{i}.v"].T).view(T, 1, d)
            h = h + llama.attention(q, k, v, 0.25).reshape(T, 2 * d) @ w[f"l{i}.o"].T
            m = llama.rms_norm(h, w[f"l{i}.n2"], 1e-5)
            expert = (m @ w[f"l{i}.r"].T).argmax(dim=1)
            hid = torch.relu(torch.einsum("th,tih->ti", m, w[f"l{i}.w1"][expert]))
            h = h + torch.einsum("ti,thi->th", hid, w[f"l{i}.w2"][expert])
        return llama.rms_norm(h, w["fn"], 1e-5) @ w["head"].T

    rng = np.random.default_rng(3)
    tokens = rng.integers(0, vocab, 41).tolist()
    want = plain(tokens)
    assert stepper.cache.admit("r")
    got, at = [], 0
    for n in (17, 2, 1, 1, 9, 1, 10):                       # a portion, tiny portions, decoded tokens
        got.append(stepper.step([StepEntry("r", tokens[at:at + n], list(range(n)))]).cpu().double())
        at += n
    # a routed layer can flip an expert on a near tie; with these seeds no row is that close
    torch.testing.assert_close(torch.cat(got), want, rtol=5e-5, atol=5e-5)


def windowed_spec(hidden=32, vocab=61, window=20):
    """Two attention layers with different cache needs: layer 0 sees all keys, layer 1 the last `window` only."""
    from tesseract_b200.config import LayerSpec, ModelSpec, PartSpec, RunEntry

    def norm(name):
        return PartSpec.make("rms_norm", {"size": hidden, "eps": 1e-5}, {"weight": name})

    def layer(i, win):
        mixer = PartSpec.make("attention", {"hidden_size": hidden, "num_heads": 4, "num_kv_heads": 2, "head_dim": 16,
                                            "window": win, "scale": None},
                              {"q": f"l{i}.q", "k": f"l{i}.k", "v": f"l{i}.v", "o": f"l{i}.o"},
                              {"position": PartSpec.make("rotary", {"head_dim": 16, "theta": 1000.0, "scaling": None})})
        ffn = PartSpec.make("swiglu", {"hidden_size": hidden, "intermediate_size": 48},
                            {"gate": f"l{i}.g", "up": f"l{i}.u", "down": f"l{i}.d"})
        return LayerSpec.make("pre_norm", mixer, ffn, {"input": norm(f"l{i}.n1"), "post_mixer": norm(f"l{i}.n2")})

    sizes = {"vocab_size": vocab, "hidden_size": hidden}
    return ModelSpec(architecture="WindowedForTests", hidden_size=hidden, vocab_size=vocab, max_positions=512,
                     embedding=PartSpec.make("token_embedding", sizes, {"table": "emb"}),
                     layers=(layer(0, None), layer(1, window)), run_order=(RunEntry(0), RunEntry(1)),
                     final_norm=norm("fn"), head=PartSpec.make("lm_head", sizes, {"weight": "head"}))


def windowed_plain(tensors, tokens, window):
    w = {k: v.double() for k, v in tensors.items()}
    T = len(tokens)
    cos, sin = llama.rope_tables(range(T), llama.rope_inverse_frequencies(16, 1000.0, None))
    h = llama.embed(tokens, w["emb"])
    for i, win in ((0, None), (1, window)):
        x = llama.rms_norm(h, w[f"l{i}.n1"], 1e-5)
        q = llama.rotate_half((x @ w[f"l{i}.q"].T).view(T, 4, 16), cos, sin)
        k = llama.rotate_half((x @ w[f"l{i}.k"].T).view(T, 2, 16), cos, sin)
        v = (x @ w[f"l{i}.v"].T).view(T, 2, 16)
        h = h + llama.attention(q, k, v, 0.25, win).reshape(T, 64) @ w[f"l{i}.o"].T
        m = llama.rms_norm(h, w[f"l{i}.n2"], 1e-5)
        h = h + llama.swiglu(m, w[f"l{i}.g"], w[f"l{i}.u"], w[f"l{i}.d"])
    return llama.rms_norm(h, w["fn"], 1e-5) @ w["head"].T


@pytest.mark.parametrize("dtype, tol", [(torch.float32, 3e-5), (torch.bfloat16, 3e-2)])
def test_layers_with_and_without_a_window_keep_pages_of_their_own(dtype, tol):
    """One model, two cache groups: the windowed layer's pages go back as the window passes them and are used
    again, the other layer keeps every page; portions and decoded tokens of three requests share the steps."""
    from tesseract_b200.engine import StepEntry, make_stepper
    from tesseract_b200.models import DecoderModel, tensor_roles

    window = 20
    spec = windowed_spec(window=window)
    g = torch.Generator().manual_seed(4)
    tensors = {name: cls.random_tensor(part, role, tuple(want.shape), g) * (4 if role in "qk" else 1)
               for cls, part, role, name, want in tensor_roles(spec)}
    model = DecoderModel(spec, {k: v.to(dtype) if v.dtype != torch.float32 or k.endswith((".q", ".k", ".v", ".o", ".g",
                                ".u", ".d", "emb", "head")) else v for k, v in tensors.items()}, runtime(dtype))
    # 11 pages of 16 tokens per group: two live requests fill the full layer's pool, the third uses pages again
    stepper = make_stepper(model, capacity_tokens=176, max_requests=3, max_step_tokens=32)
    cache = stepper.cache
    assert len(cache.groups) == 2
    windowed = [i for i, grp in enumerate(cache.groups) if grp.need.window][0]
    rng = np.random.default_rng(7)
    seqs = {"a": rng.integers(0, 61, 90).tolist(), "b": rng.integers(0, 61, 70).tolist(),
            "c": rng.integers(0, 61, 78).tolist()}
    rounded = {k: v.to(dtype).float() for k, v in tensors.items()}
    plain = {r: windowed_plain(rounded, t, window) for r, t in seqs.items()}
    got = {r: [] for r in seqs}
    at = {r: 0 for r in seqs}
    sizes = [16, 7, 2, 5, 1, 1, 23, 1, 3]
    live, waiting, step = [], ["a", "b", "c"], 0
    peak_windowed = 0
    while live or waiting:
        while waiting and len(live) < 2 and cache.admit(waiting[0], None):
            live.append(waiting.pop(0))
        entries = []
        for j, r in enumerate(live):
            n = min(sizes[(step + 3 * j) % len(sizes)], len(seqs[r]) - at[r])
            entries.append(StepEntry(r, seqs[r][at[r]:at[r] + n], list(range(n))))
            at[r] += n
        logits = stepper.step(entries).cpu().double()
        k = 0
        for e in entries:
            got[e.request].append(logits[k:k + len(e.tokens)])
            k += len(e.tokens)
        cache.check()
        for r in live:
            held = len(cache.pages_of(r, windowed))
            peak_windowed = max(peak_windowed, held)
            assert len(cache.pages_of(r, 1 - windowed)) == -(-at[r] // 16)          # the full layer keeps every page
        for r in [r for r in live if at[r] == len(seqs[r])]:
            cache.release(r)
            live.remove(r)
        step += 1
    assert peak_windowed <= -(-(window - 1 + 32) // 16) + 1                          # the window bounds what is held
    assert cache.pages_reused > 0 and cache.used_pages() == 0
    for r in seqs:
        torch.testing.assert_close(torch.cat(got[r]), plain[r], rtol=tol, atol=tol)


@pytest.mark.parametrize("nh, nkv, d", [(8, 2, 64), (6, 2, 128)])
def test_attention_part_with_the_tcgen05_prompt_kernel(nh, nkv, d):
    """The same mixer with prompt portions on the tcgen05 kernel: portions, decode rows beside them, page reuse."""
    from tesseract_b200 import kernels
    from tesseract_b200.cache import CacheManager
    from tesseract_b200.config import PartSpec
    from tesseract_b200.parts import MIXERS

    torch.manual_seed(3)
    rt = runtime(torch.bfloat16)
    hidden = 128
    position = PartSpec.make("rotary", {"head_dim": d, "theta": 10000.0, "scaling": None})
    weights = {"q": torch.randn(nh * d, hidden) * 0.1, "k": torch.randn(nkv * d, hidden) * 0.1,
               "v": torch.randn(nkv * d, hidden) * 0.1, "o": torch.randn(hidden, nh * d) * 0.1}
    weights = {k: v.to(torch.bfloat16) for k, v in weights.items()}
    outs = {}
    for kernel in ("mma", "tcgen05"):
        spec = PartSpec.make("attention", {"hidden_size": hidden, "num_heads": nh, "num_kv_heads": nkv, "head_dim": d,
                                           "window": None, "scale": None, "prompt_kernel": kernel},
                             {"q": "q", "k": "k", "v": "v", "o": "o"}, {"position": position})
        mixer = MIXERS.get("attention")(spec, weights, rt)
        cache = CacheManager([mixer.cache_need()], [None], num_pages=40, page_size=16, max_requests=2,
                             dtype=torch.bfloat16, device=rt.device, max_step_tokens=256)
        gen = torch.Generator().manual_seed(5)
        xs = {"a": torch.randn(300, hidden, generator=gen).to(torch.bfloat16),
              "b": torch.randn(140, hidden, generator=gen).to(torch.bfloat16)}
        cuts = {"a": [130, 169, 1], "b": [1, 138, 1]}
        got = {"a": [], "b": []}
        for r in xs:
            assert cache.admit(r)
        for step in range(3):
            news = [cuts[r][step] for r in ("a", "b")]
            for r, n in zip(("a", "b"), news):
                cache.extend(r, n)
            ctx = context_for(cache, ["a", "b"], news)
            x = torch.cat([xs[r][cache.length(r):cache.length(r) + n] for r, n in zip(("a", "b"), news)]).cuda()
            y = mixer.forward(x, ctx, cache.bindings[0]).cpu()
            at = 0
            for r, n in zip(("a", "b"), news):
                got[r].append(y[at:at + n])
                at += n
                cache.commit(r, n)
        outs[kernel] = {r: torch.cat(v).float() for r, v in got.items()}
        assert kernels.tcgen05_error() == 0
    for r in ("a", "b"):
        torch.testing.assert_close(outs["tcgen05"][r], outs["mma"][r], rtol=3e-2, atol=3e-2)
