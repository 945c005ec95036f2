"""A mixer with state of its own, defined here, is registered, built and stepped
without any change to the framework: the cache manager gives it a state slot, the
step function carries the state across portions, and the model runs it in a layer of
its own beside an attention layer.  The order list also runs one layer twice and lets
a run read another run's cache."""

import json
from dataclasses import dataclass

import pytest
import torch

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu
DEV = "cuda"
D_MODEL, HEADS, KV, HD, FF, VOCAB = 48, 4, 2, 16, 80, 120


def make_toy():
    from socrates_b200.cache import CacheNeeds, StateSpec
    from socrates_b200.parts import Branch, ParamSpec, Part

    class DecayMixer(Part):
        """s_t = decay * s_{t-1} + x_t per request; output W s_t.  The state s lives in
        the request's state slot."""
        supports_graph = False          # it walks the host-side batch

        def __init__(self, spec, name):
            super().__init__(spec, name)
            self.d = spec.params["hidden_size"]
            self.decay = spec.params["decay"]

        def parameters(self):
            return {self.name + "proj.weight": ParamSpec((self.d, self.d))}

        def bind(self, tensors, dtype):
            self.w = tensors[self.name + "proj.weight"]

        def cache_needs(self):
            return CacheNeeds(state=StateSpec((self.d,), torch.float32))

        def forward(self, ctx, x, cache):
            state = cache.state()
            out = torch.empty(x.shape, dtype=torch.float32, device=x.device)
            i = 0
            for e in ctx.host_batch:
                s = state[e.row]
                for _ in e.tokens:
                    s = self.decay * s + x[i].float()
                    out[i] = s
                    i += 1
                state[e.row] = s
            return Branch((out @ self.w.float().T).unsqueeze(0).contiguous())

    return DecayMixer


@dataclass(frozen=True)
class ToyConfig:
    decay: float = 0.9
    architecture = "ToyDecayForCausalLM"

    @classmethod
    def from_dict(cls, d):
        return cls(decay=float(d["decay"]))

    def to_dict(self):
        return {"architectures": [self.architecture], "decay": self.decay, "vocab_size": VOCAB}

    def plan(self):
        from socrates_b200.config import LayerSpec, ModelPlan, PartSpec, RunEntry
        norm = {"dim": D_MODEL, "eps": 1e-5}
        norms = (PartSpec("rmsnorm", norm, "n1."), PartSpec("rmsnorm", norm, "n2."))
        ff = PartSpec("swiglu", {"hidden_size": D_MODEL, "intermediate_size": FF}, "mlp.")
        attn = PartSpec("gqa_attention", {
            "hidden_size": D_MODEL, "num_heads": HEADS, "num_kv_heads": KV, "head_dim": HD,
            "scale": HD ** -0.5, "qk_norm_eps": 1e-5, "window": None,
            "position": PartSpec("rotary", {"head_dim": HD, "rotary_dim": HD, "theta": 1e4})}, "attn.")
        toy = PartSpec("toy_decay", {"hidden_size": D_MODEL, "decay": self.decay}, "mix.")
        layers = (LayerSpec("pre_norm", "layers.0.", norms, toy, ff),
                  LayerSpec("pre_norm", "layers.1.", norms, attn, ff))
        # layer 0 (state), layer 1 (attention), layer 1 again with a cache of its own,
        # layer 1 once more reading the cache of its first run, then layer 0 again.
        order = (RunEntry(0), RunEntry(1), RunEntry(1), RunEntry(1, reads_cache_of=1), RunEntry(0))
        return ModelPlan(self.architecture, D_MODEL, VOCAB,
                         PartSpec("embedding", {"vocab_size": VOCAB, "hidden_size": D_MODEL}, "embed."),
                         layers, order, PartSpec("rmsnorm", norm, "norm."),
                         PartSpec("lm_head", {"hidden_size": D_MODEL, "vocab_size": VOCAB, "tied_to": None}, "head."))


def plain_toy(w, ids, decay):
    """Whole-sequence statement of the toy model with the plain implementation's functions."""
    w = {k: v.double() for k, v in w.items()}
    cfg = {"num_attention_heads": HEADS, "num_key_value_heads": KV, "head_dim": HD, "rms_norm_eps": 1e-5,
           "rope_theta": 1e4}
    T = len(ids)
    pos = torch.arange(T)
    x = w["embed.weight"][torch.tensor(ids)]

    def toy_layer(x):
        h = plain.rms_norm(x, w["layers.0.n1.weight"], 1e-5)
        s, outs = torch.zeros(D_MODEL, dtype=torch.float64), []
        for t in range(T):
            s = decay * s + h[t]
            outs.append(s)
        x = x + torch.stack(outs) @ w["layers.0.mix.proj.weight"].T
        return x + plain.swiglu(plain.rms_norm(x, w["layers.0.n2.weight"], 1e-5), w, "layers.0.mlp.")

    def attn_layer(x, kv_from=None):
        h = plain.rms_norm(x, w["layers.1.n1.weight"], 1e-5)
        p = "layers.1.attn."
        q = (h @ w[p + "q_proj.weight"].T).view(T, HEADS, HD)
        src = h if kv_from is None else kv_from
        k = (src @ w[p + "k_proj.weight"].T).view(T, KV, HD)
        v = (src @ w[p + "v_proj.weight"].T).view(T, KV, HD)
        cos, sin = plain.rope_tables(pos, HD, 1e4)
        q = plain.apply_rope(plain.rms_norm(q, w[p + "q_norm.weight"], 1e-5), cos, sin)
        k = plain.apply_rope(plain.rms_norm(k, w[p + "k_norm.weight"], 1e-5), cos, sin)
        o = plain.attention_core(q, k, v, HD ** -0.5, plain.attention_mask(pos, pos, None))
        x = x + o.reshape(T, HEADS * HD) @ w[p + "o_proj.weight"].T
        return x + plain.swiglu(plain.rms_norm(x, w["layers.1.n2.weight"], 1e-5), w, "layers.1.mlp."), h

    x = toy_layer(x)
    x, h_first = attn_layer(x)
    x, _ = attn_layer(x)
    x, _ = attn_layer(x, kv_from=h_first)          # reads the keys and values of the first attention run
    x = toy_layer(x)
    return plain.rms_norm(x, w["norm.weight"], 1e-5) @ w["head.weight"].T


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.bfloat16, 3e-2)])
def test_toy_mixer_with_state_registers_builds_and_steps(tmp_path, dtype, tol):
    from safetensors.torch import load_file
    from socrates_b200.cache import CacheManager
    from socrates_b200.config import register_architecture, unregister_architecture
    from socrates_b200.engine.engine import build_model
    from socrates_b200.engine.runner import ModelRunner, StepEntry
    from socrates_b200.parts import register_part, unregister_part
    from socrates_b200.weights import write_model_folder

    register_part("mixer", "toy_decay", make_toy())
    register_architecture(ToyConfig.architecture, ToyConfig)
    try:
        folder = write_model_folder(ToyConfig(0.9), seed=4, out_dir=tmp_path / "toy")
        assert json.loads((folder / "config.json").read_text())["architectures"] == [ToyConfig.architecture]
        w = load_file(str(folder / "model.safetensors"))
        config, model = build_model(folder, dtype, DEV)
        assert isinstance(config, ToyConfig) and not model.supports_graph
        needs = model.cache_needs()
        assert needs[0].state is not None and needs[0].paged is None and needs[3] is None
        cache = CacheManager(needs, 3, 128, 16, 12, dtype, DEV)
        assert len(cache.groups) == 1 and cache.groups[0].entries == [1, 2] and set(cache.states) == {0, 4}
        runner = ModelRunner(model, cache, dtype, DEV, max_tokens=128, max_seqs=3)

        g = torch.Generator().manual_seed(0)
        seqs = [torch.randint(0, VOCAB, (n,), generator=g).tolist() for n in (41, 18)]
        want = [plain_toy(w, s, 0.9) for s in seqs]
        got = [[], []]
        fed = [0, 0]
        for r in (0, 1):
            cache.assign(r)
        # request 0 in portions of 7, 2, 20, then one by one; request 1 joins late, then both decode
        plan = [[(0, 7)], [(0, 2)], [(0, 20), (1, 5)], [(0, 1), (1, 11)], [(0, 1), (1, 1)], [(0, 1), (1, 1)]]
        while fed[0] < 41:
            step = plan.pop(0) if plan else [(0, 1)]
            entries = []
            for r, c in step:
                c = min(c, len(seqs[r]) - fed[r])
                if c <= 0:
                    continue
                assert cache.reserve(r, fed[r] + c)
                entries.append(StepEntry(r, seqs[r][fed[r]:fed[r] + c], fed[r], list(range(c))))
            logits = runner.step(entries).logits.double().cpu()
            i = 0
            for e in entries:
                n = len(e.tokens)
                got[e.row].append(logits[i:i + n])
                i += n
                fed[e.row] += n
                cache.commit(e.row, fed[e.row])
        for r in (0, 1):
            mine = torch.cat(got[r])
            ref = want[r][:mine.shape[0]]
            assert float((mine - ref).abs().max() / ref.abs().max()) < tol
        # a new request in a used row starts from a zeroed state
        cache.release(1)
        cache.assign(1)
        assert cache.reserve(1, 4)
        logits = runner.step([StepEntry(1, seqs[0][:4], 0, [3])]).logits.double().cpu()
        assert float((logits[0] - want[0][3]).abs().max() / want[0].abs().max()) < tol
    finally:
        unregister_part("mixer", "toy_decay")
        unregister_architecture(ToyConfig.architecture)


def test_toy_mixer_with_state_through_the_entry_point(tmp_path):
    """The same mixer through Engine with running ahead switched on.  A step that is launched
    early and then dropped would advance the state slots a second time when it is run again, so
    the engine must not run ahead for a model that keeps per-request state.  Requests of
    different lengths end at different steps (each end would drop an early step); every produced
    token is checked against the whole-sequence statement."""
    from safetensors.torch import load_file
    from socrates_b200 import Engine
    from socrates_b200.config import register_architecture, unregister_architecture
    from socrates_b200.parts import register_part, unregister_part
    from socrates_b200.weights import write_model_folder

    register_part("mixer", "toy_decay", make_toy())
    register_architecture(ToyConfig.architecture, ToyConfig)
    try:
        folder = write_model_folder(ToyConfig(0.9), seed=4, out_dir=tmp_path / "toy")
        w = load_file(str(folder / "model.safetensors"))
        g = torch.Generator().manual_seed(1)
        prompts = [torch.randint(0, VOCAB, (n,), generator=g).tolist() for n in (9, 21, 4, 15)]
        new = [12, 5, 17, 8]
        eng = Engine(str(folder), device="cuda:0", dtype="float32", max_batch=3, max_len=64, max_new_tokens=20,
                     token_budget=16, run_ahead=True)
        reqs = [eng.submit(p, max_new_tokens=n) for p, n in zip(prompts, new)]
        while eng.scheduler.has_work():
            assert eng.step()
            eng.scheduler.check()
        assert eng.ahead_launched == 0                       # state slots: no step is launched early
        for p, n, r in zip(prompts, new, reqs):
            assert r.done and len(r.output) == n
            logits = plain_toy(w, list(p) + r.output[:-1], 0.9)
            scale = float(logits.abs().max())
            for i, tok in enumerate(r.output):
                row = logits[len(p) - 1 + i]
                best = int(torch.argmax(row))
                assert tok == best or float(row[best] - row[tok]) <= 1e-4 * scale, (i, tok, best)
    finally:
        unregister_part("mixer", "toy_decay")
        unregister_architecture(ToyConfig.architecture)


# ------------------------------------------------------------------------------------------
# A feed-forward with routing and another position encoding, defined here.

E_EXPERTS, E_FF = 3, 40


def make_routed():
    from socrates_b200.parts import Branch, ParamSpec, Part
    from socrates_b200.parts.linear import Linear

    class RoutedFF(Part):
        """Top-1 of E experts per token: router logits and their softmax in float32, tokens
        gathered per expert, each expert up -> SiLU -> down through the engine's own products,
        outputs scattered back times the router's probability."""
        supports_graph = False          # how many tokens an expert gets is known on the host only

        def __init__(self, spec, name):
            super().__init__(spec, name)
            self.d, self.f, self.E = spec.params["hidden_size"], spec.params["expert_size"], spec.params["experts"]

        def parameters(self):
            # role "gain": held as float32 on the device whatever the model dtype is
            p = {self.name + "router.weight": ParamSpec((self.E, self.d), role="gain", init="normal")}
            for e in range(self.E):
                p[f"{self.name}experts.{e}.up.weight"] = ParamSpec((self.f, self.d))
                p[f"{self.name}experts.{e}.down.weight"] = ParamSpec((self.d, self.f))
            return p

        def bind(self, tensors, dtype):
            self.router = tensors[self.name + "router.weight"].float()
            self.up = [Linear(tensors[f"{self.name}experts.{e}.up.weight"]) for e in range(self.E)]
            self.down = [Linear(tensors[f"{self.name}experts.{e}.down.weight"]) for e in range(self.E)]

        def forward(self, ctx, x):
            probs = torch.softmax(x.float() @ self.router.T, dim=-1)          # float32
            top_p, top_e = probs.max(dim=-1)
            out = torch.zeros(1, x.shape[0], self.d, dtype=torch.float32, device=x.device)
            for e in range(self.E):
                rows = (top_e == e).nonzero().flatten()
                if rows.numel() == 0:
                    continue
                xe = x.index_select(0, rows).contiguous()
                h = self.up[e](ctx, xe, f"toy_up{e}", out="float32")
                h = (h * torch.sigmoid(h)).to(x.dtype)
                y = self.down[e](ctx, h, f"toy_down{e}", out="float32")
                out[0].index_copy_(0, rows, y * top_p[rows, None])
            return Branch(out)

    return RoutedFF


def make_linear_position():
    from socrates_b200.parts import Part

    class LinearFrequencies(Part):
        """Frequencies that fall linearly, not geometrically, over the first `rotary_dim` dims."""

        def __init__(self, spec, name=""):
            super().__init__(spec, name)
            self.rotary_dim, self.top = int(spec.params["rotary_dim"]), float(spec.params["top"])
            self._table = None

        def inv_freq(self):
            n = self.rotary_dim // 2
            return self.top * (1.0 - torch.arange(n).float() / n)

        def tables(self, device):
            if self._table is None:
                self._table = self.inv_freq().to(device=device, dtype=torch.float32).contiguous()
            return self._table, self.rotary_dim

    return LinearFrequencies


@dataclass(frozen=True)
class RoutedConfig:
    architecture = "ToyRoutedForCausalLM"

    @classmethod
    def from_dict(cls, d):
        return cls()

    def to_dict(self):
        return {"architectures": [self.architecture], "vocab_size": VOCAB}

    def plan(self):
        from socrates_b200.config import LayerSpec, ModelPlan, PartSpec, RunEntry
        norm = {"dim": D_MODEL, "eps": 1e-5}
        norms = (PartSpec("rmsnorm", norm, "n1."), PartSpec("rmsnorm", norm, "n2."))

        def attn(position):
            return PartSpec("gqa_attention", {
                "hidden_size": D_MODEL, "num_heads": HEADS, "num_kv_heads": KV, "head_dim": HD,
                "scale": HD ** -0.5, "qk_norm_eps": None, "window": None, "position": position}, "attn.")
        routed = PartSpec("toy_routed", {"hidden_size": D_MODEL, "expert_size": E_FF, "experts": E_EXPERTS}, "moe.")
        dense = PartSpec("swiglu", {"hidden_size": D_MODEL, "intermediate_size": FF}, "mlp.")
        layers = (LayerSpec("pre_norm", "layers.0.", norms,
                            attn(PartSpec("toy_linear_freq", {"rotary_dim": 8, "top": 0.5})), routed),
                  LayerSpec("pre_norm", "layers.1.", norms,
                            attn(PartSpec("rotary", {"head_dim": HD, "rotary_dim": 12, "theta": 1e3})), dense))
        return ModelPlan(self.architecture, D_MODEL, VOCAB,
                         PartSpec("embedding", {"vocab_size": VOCAB, "hidden_size": D_MODEL}, "embed."),
                         layers, (RunEntry(0), RunEntry(1)), PartSpec("rmsnorm", norm, "norm."),
                         PartSpec("lm_head", {"hidden_size": D_MODEL, "vocab_size": VOCAB, "tied_to": "embed.weight"},
                                  "head."))


def plain_routed(w, ids):
    w = {k: v.double() for k, v in w.items()}
    T = len(ids)
    pos = torch.arange(T)
    x = w["embed.weight"][torch.tensor(ids)]

    def rotate(t, inv_freq, R):
        ang = pos[:, None].double() * inv_freq[None, :].double()
        cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        a, b, rest = t[..., :R // 2], t[..., R // 2:R], t[..., R:]
        return torch.cat([a * cos - b * sin, b * cos + a * sin, rest], dim=-1)

    def attention(x, i, inv_freq, R):
        p = f"layers.{i}.attn."
        h = plain.rms_norm(x, w[f"layers.{i}.n1.weight"], 1e-5)
        q = rotate((h @ w[p + "q_proj.weight"].T).view(T, HEADS, HD), inv_freq, R)
        k = rotate((h @ w[p + "k_proj.weight"].T).view(T, KV, HD), inv_freq, R)
        v = (h @ w[p + "v_proj.weight"].T).view(T, KV, HD)
        o = plain.attention_core(q, k, v, HD ** -0.5, plain.attention_mask(pos, pos, None))
        return x + o.reshape(T, HEADS * HD) @ w[p + "o_proj.weight"].T

    x = attention(x, 0, 0.5 * (1.0 - torch.arange(4).float() / 4), 8)
    h = plain.rms_norm(x, w["layers.0.n2.weight"], 1e-5)
    probs = torch.softmax(h @ w["layers.0.moe.router.weight"].T, dim=-1)
    top_p, top_e = probs.max(dim=-1)
    y = torch.zeros_like(x)
    for t in range(T):
        e = int(top_e[t])
        u = h[t] @ w[f"layers.0.moe.experts.{e}.up.weight"].T
        y[t] = top_p[t] * ((u * torch.sigmoid(u)) @ w[f"layers.0.moe.experts.{e}.down.weight"].T)
    x = x + y
    x = attention(x, 1, 1.0 / (1e3 ** (torch.arange(0, 12, 2).float() / 12)), 12)
    x = x + plain.swiglu(plain.rms_norm(x, w["layers.1.n2.weight"], 1e-5), w, "layers.1.mlp.")
    return plain.rms_norm(x, w["norm.weight"], 1e-5) @ w["embed.weight"].T


def test_toy_routed_feed_forward_and_position_encoding(tmp_path):
    """A routed feed-forward and a position encoding of its own, registered from here: one
    layer uses both, the next the built-in rotation over 12 of 16 dims (a rotation that is
    neither all dims nor none) and no QK norm; float32, prompt portions then single tokens."""
    from safetensors.torch import load_file
    from socrates_b200.cache import CacheManager
    from socrates_b200.config import register_architecture, unregister_architecture
    from socrates_b200.engine.engine import build_model
    from socrates_b200.engine.runner import ModelRunner, StepEntry
    from socrates_b200.parts import register_part, unregister_part
    from socrates_b200.weights import write_model_folder

    register_part("feed_forward", "toy_routed", make_routed())
    register_part("position", "toy_linear_freq", make_linear_position())
    register_architecture(RoutedConfig.architecture, RoutedConfig)
    try:
        folder = write_model_folder(RoutedConfig(), seed=9, out_dir=tmp_path / "routed")
        w = load_file(str(folder / "model.safetensors"))
        config, model = build_model(folder, torch.float32, DEV)
        assert not model.supports_graph
        assert model.layers[0].feed_forward.router.dtype == torch.float32
        cache = CacheManager(model.cache_needs(), 2, 128, 16, 10, torch.float32, DEV)
        runner = ModelRunner(model, cache, torch.float32, DEV, max_tokens=64, max_seqs=2)
        ids = torch.randint(0, VOCAB, (37,), generator=torch.Generator().manual_seed(2)).tolist()
        want = plain_routed(w, ids)
        experts_used = set()
        cache.assign(0)
        got, fed = [], 0
        for count in (9, 2, 16, 1, 1, 1, 7):
            assert cache.reserve(0, fed + count)
            logits = runner.step([StepEntry(0, ids[fed:fed + count], fed, list(range(count)))]).logits
            got.append(logits.double().cpu())
            fed += count
            cache.commit(0, fed)
        mine = torch.cat(got)
        assert float((mine - want).abs().max() / want.abs().max()) < 1e-4
        h = plain.rms_norm(w["embed.weight"].double()[torch.tensor(ids)], torch.ones(D_MODEL, dtype=torch.float64), 1e-5)
        experts_used = set(torch.softmax(h @ w["layers.0.moe.router.weight"].double().T, -1).argmax(-1).tolist())
        assert len(experts_used) >= 2, "the random router sent every token to one expert: the test shows nothing"
    finally:
        unregister_part("feed_forward", "toy_routed")
        unregister_part("position", "toy_linear_freq")
        unregister_architecture(RoutedConfig.architecture)
