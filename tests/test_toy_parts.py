"""A mixer with state of its own, a feed-forward that routes every token to one of three experts, a
position encoding with stretched positions and another that turns neighbouring features by angles from
a table, a run order that names a layer twice, and an entry that reads another entry's cache: all defined HERE, registered, built and stepped through the
framework's own model, cache and step function without touching its files. The toy is no one's model."""
import json
from dataclasses import dataclass

import numpy as np
import pytest
import torch

import helpers
import plain_qwen3 as plain
import torch_ops
from tinyinfer_b200.config import (AttentionSpec, ExecStep, GatedMLPSpec, LayerSpec, ModelSpec, NormSpec,
                                   PositionSpec, TensorNames, register_architecture)
from tinyinfer_b200.models import DecoderModel
from tinyinfer_b200.parts import (FeedForward, Mixer, PositionEncoding, StateNeed, TensorSpec,
                                  register_feed_forward, register_mixer, register_position)


# ------------------------------------------------------------------ the toy, as a user would write it
@dataclass(frozen=True)
class RunningMeanSpec:
    hidden_size: int
    kind: str = "toy_running_mean"


class RunningMeanMixer(Mixer):
    """out[t] = mean over the request's tokens 0..t of (x W^T). Its state, one float32 vector per
    request, is the sum so far; it keeps no pages."""

    def tensors(self):
        h = self.spec.hidden_size
        return {"proj.weight": TensorSpec((h, h))}

    def load(self, tensors):
        self.w = tensors["proj.weight"]

    def state_need(self):
        return StateNeed((self.spec.hidden_size,), torch.float32)

    def forward(self, x, step, cache):
        y = (x.float() @ self.w.float().T)
        out = torch.empty_like(y)
        row = 0
        for i, (n, start) in enumerate(zip(step.q_lens, step.starts)):
            slot = int(step.state_slots[i])
            running = cache.state[slot] + torch.cumsum(y[row:row + n], dim=0)
            counts = torch.arange(start + 1, start + n + 1, device=y.device, dtype=torch.float32)[:, None]
            out[row:row + n] = running / counts
            cache.state[slot] = running[-1]
            row += n
        return out.to(x.dtype)


register_mixer("toy_running_mean", RunningMeanMixer)


class RunningMeanOnDevice(RunningMeanMixer):
    """The same mixer with nothing read on the host: the state slots, the rows' requests and positions
    are used where they lie, on the device, so a step of single tokens can be captured in a CUDA graph
    and replayed (``graph_safe``). Rows that only fill a batch up to its graph's size carry a slot of
    their own that no request holds."""
    graph_safe = True

    def forward(self, x, step, cache):
        y = (x.float() @ self.w.float().T).double()
        seq, slots, cu = step.token_seq.long(), step.state_slots.long(), step.cu_seqlens.long()
        sums = torch.cat((torch.zeros_like(y[:1]), torch.cumsum(y, dim=0)))       # sums[r]: of the rows before r
        running = cache.state.index_select(0, slots).double()[seq] + sums[1:] - sums[cu[:-1]][seq]
        cache.state.index_copy_(0, slots, running[cu[1:] - 1].float())
        return (running / (step.positions.double() + 1.0)[:, None]).to(x.dtype)


register_mixer("toy_running_mean_on_device", RunningMeanOnDevice)


@dataclass(frozen=True)
class RoutedSpec:
    hidden_size: int
    intermediate_size: int
    num_experts: int
    kind: str = "toy_top1_experts"


class RoutedFeedForward(FeedForward):
    """Every token goes to the one expert its router logit (float32) is largest for; the expert is a
    gated MLP whose output is scaled by the softmax weight of that logit. Built from the package's
    own products; the routing itself is plain tensor code, which is all a toy needs."""

    def tensors(self):
        h, i, e = self.spec.hidden_size, self.spec.intermediate_size, self.spec.num_experts
        t = {"router.weight": TensorSpec((e, h), role="vector32")}
        for k in range(e):
            t[f"experts.{k}.gate_up.weight"] = TensorSpec((2 * i, h))
            t[f"experts.{k}.down.weight"] = TensorSpec((h, i))
        return t

    def load(self, tensors):
        self.w = tensors

    def forward(self, x, step):
        from tinyinfer_b200 import ops
        logits = x.float() @ self.w["router.weight"].T
        weight, choice = torch.softmax(logits, dim=-1).max(dim=-1)
        out = torch.zeros_like(x)
        for k in range(self.spec.num_experts):
            rows = (choice == k).nonzero().flatten()
            if rows.numel() == 0:
                continue
            hidden = ops.gated_linear(x.index_select(0, rows).contiguous(), self.w[f"experts.{k}.gate_up.weight"])
            y = ops.linear(hidden, self.w[f"experts.{k}.down.weight"])
            out.index_copy_(0, rows, (y.float() * weight[rows, None]).to(x.dtype))
        return out


register_feed_forward("toy_top1_experts", RoutedFeedForward)


class RoutedOnDevice(RoutedFeedForward):
    """The same feed-forward with no row picked on the host: every expert runs on every token and each
    token keeps its own expert's answer (a row of a product does not depend on the rows beside it), which
    is wasteful and may be captured in a CUDA graph."""
    graph_safe = True

    def forward(self, x, step):
        from tinyinfer_b200 import ops
        logits = x.float() @ self.w["router.weight"].T
        weight, choice = torch.softmax(logits, dim=-1).max(dim=-1)
        out = torch.zeros_like(x)
        for k in range(self.spec.num_experts):
            y = ops.linear(ops.gated_linear(x, self.w[f"experts.{k}.gate_up.weight"]), self.w[f"experts.{k}.down.weight"])
            out = torch.where((choice == k)[:, None], (y.float() * weight[:, None]).to(x.dtype), out)
        return out


register_feed_forward("toy_top1_experts_on_device", RoutedOnDevice)


@dataclass(frozen=True)
class StretchedRopeSpec:
    theta: float
    rotary_dim: int
    stretch: float                     # position p turns as position p / stretch would
    kind: str = "toy_stretched_rope"


class StretchedRope(PositionEncoding):
    """Rotary encoding with every position divided by a constant: the same rotation kernel, other
    frequencies. The attention mixer asks its position part only for inv_freq and rotary_dim."""

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        exponent = torch.arange(0, spec.rotary_dim, 2, dtype=torch.float32) / spec.rotary_dim
        self.inv_freq = (1.0 / (spec.theta ** exponent) / spec.stretch).to(device)
        self.rotary_dim = spec.rotary_dim


register_position("toy_stretched_rope", StretchedRope)


@dataclass(frozen=True)
class PairTableRopeSpec:
    theta: float
    rotary_dim: int                    # may be less than the head size: the rest of a head is not turned
    max_positions: int
    kind: str = "toy_pair_table_rope"


def pair_table_angles(theta, rotary_dim, positions, dtype):
    """angle[p][j] = 4 * log(1 + p) * theta ** (-2j / rotary_dim): no inverse frequencies give this law."""
    freq = theta ** (-torch.arange(0, rotary_dim, 2, dtype=dtype) / rotary_dim)
    return 4.0 * torch.log1p(torch.as_tensor(positions, dtype=dtype))[:, None] * freq[None, :]


class PairTableRope(PositionEncoding):
    """Neighbouring features (2j, 2j + 1) form a pair, and a pair's angle at a position stands in a table
    of cosines and sines: what the part hands to its mixer is an ``ops.Rotation`` that says so. The mixer
    and the fused kernel are the framework's own, unchanged."""

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        ang = pair_table_angles(spec.theta, spec.rotary_dim, range(spec.max_positions), torch.float32)
        self.table = torch.cat((ang.cos(), ang.sin()), dim=1).contiguous().to(device)

    def rotation(self):
        from tinyinfer_b200 import ops
        return ops.Rotation(self.spec.rotary_dim, cos_sin=self.table, interleaved=True)


register_position("toy_pair_table_rope", PairTableRope)

TOY = dict(architectures=["ToyForCausalLM"], vocab_size=97, hidden_size=48, heads=3, kv_heads=1, head_dim=16,
           intermediate_size=80, eps=1e-5, theta=10000.0, max_positions=256, experts=3, expert_size=24, stretch=4.0,
           position="stretched")
TOY_PAIRS = dict(TOY, position="pairs_from_table", rotary_dim=12)
TOY_ON_DEVICE = dict(TOY, state="on_device")
TOY_FRAMED = dict(TOY, architectures=["ToyFramedForCausalLM"], embedding_scale=3.0, logit_cap=2.5)


class ToyConfig:
    def __init__(self, d):
        self.d = dict(d)
        self.architectures = d["architectures"]

    @classmethod
    def from_dict(cls, d):
        return cls(d)

    def to_dict(self):
        return dict(self.d)

    def model_spec(self):
        d = self.d
        h, eps = d["hidden_size"], d["eps"]
        position = (StretchedRopeSpec(d["theta"], d["head_dim"], d["stretch"]) if d["position"] == "stretched"
                    else PairTableRopeSpec(d["theta"], d["rotary_dim"], d["max_positions"]))
        attn = AttentionSpec(h, d["heads"], d["kv_heads"], d["head_dim"], d["head_dim"] ** -0.5, position,
                             qk_norm=NormSpec(d["head_dim"], eps))
        ffn = GatedMLPSpec(h, d["intermediate_size"])
        on_device = d.get("state") == "on_device"
        routed = RoutedSpec(h, d["expert_size"], d["experts"], "toy_top1_experts_on_device" if on_device else "toy_top1_experts")
        norm = NormSpec(h, eps)
        mean = RunningMeanSpec(h, "toy_running_mean_on_device" if on_device else "toy_running_mean")
        layers = (LayerSpec(attn, ffn, norm, norm), LayerSpec(mean, routed, norm, norm))
        # layer 0 runs three times: with a cache of its own, again with another cache, and at the
        # end reading the keys its first run wrote; the stateful toy layer sits in between
        execution = (ExecStep(0, 0), ExecStep(1, 1), ExecStep(0, 2), ExecStep(0, 0, writes_cache=False))
        return ModelSpec(d["architectures"][0], d["vocab_size"], h, layers, execution, norm,
                         tie_embeddings=True, max_positions=d["max_positions"], names=TensorNames())


register_architecture("ToyForCausalLM", ToyConfig, lambda cfg, dtype, device: DecoderModel(cfg.model_spec(), dtype, device))


class FramedToyModel(DecoderModel):
    """Another frame around the same blocks: the embedding is scaled and the logits are capped smoothly.
    The model class of an architecture is whatever its registration names."""

    def __init__(self, cfg, dtype, device):
        super().__init__(cfg.model_spec(), dtype, device)
        self.scale, self.cap = cfg.d["embedding_scale"], cfg.d["logit_cap"]

    def embed(self, step):
        return (super().embed(step).float() * self.scale).to(self.dtype)

    def logits(self, x, step):
        return self.cap * torch.tanh(super().logits(x, step) / self.cap)


register_architecture("ToyFramedForCausalLM", ToyConfig, FramedToyModel)


# ------------------------------------------------------------------ its plain statement
def toy_plain(w, tokens, d=TOY):
    pos = [i / d["stretch"] for i in range(len(tokens))]
    t = len(tokens)

    def turn(a):
        """[T, heads, head_dim] turned by the toy's position encoding."""
        if d["position"] == "stretched":
            return plain.rope(a, pos, d["theta"])
        rd = d["rotary_dim"]
        ang = pair_table_angles(d["theta"], rd, range(t), a.dtype)
        cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
        even, odd = a[..., 0:rd:2], a[..., 1:rd:2]
        turned = torch.stack((even * cos - odd * sin, odd * cos + even * sin), dim=-1).flatten(-2)
        return torch.cat((turned, a[..., rd:]), dim=-1)

    def attn_layer(x, kv_from=None):
        p = "model.layers.0."
        hn = plain.rmsnorm(x, w[p + "input_layernorm.weight"], d["eps"])
        src = hn if kv_from is None else kv_from
        q = (hn @ w[p + "self_attn.q_proj.weight"].T).view(t, d["heads"], d["head_dim"])
        k = (src @ w[p + "self_attn.k_proj.weight"].T).view(t, d["kv_heads"], d["head_dim"])
        v = (src @ w[p + "self_attn.v_proj.weight"].T).view(t, d["kv_heads"], d["head_dim"])
        q = turn(plain.rmsnorm(q, w[p + "self_attn.q_norm.weight"], d["eps"]))
        k = turn(plain.rmsnorm(k, w[p + "self_attn.k_norm.weight"], d["eps"]))
        o = plain.attention(q, k, v, d["head_dim"] ** -0.5).reshape(t, -1) @ w[p + "self_attn.o_proj.weight"].T
        x = x + o
        hn2 = plain.rmsnorm(x, w[p + "post_attention_layernorm.weight"], d["eps"])
        return x + plain.swiglu(hn2, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                                w[p + "mlp.down_proj.weight"]), hn

    x = plain.embedding(tokens, w["model.embed_tokens.weight"]) * d.get("embedding_scale", 1.0)
    x, first_normed = attn_layer(x)
    p = "model.layers.1."
    hn = plain.rmsnorm(x, w[p + "input_layernorm.weight"], d["eps"])
    y = hn @ w[p + "self_attn.proj.weight"].T
    x = x + torch.cumsum(y, 0) / torch.arange(1, t + 1, dtype=x.dtype)[:, None]
    hn = plain.rmsnorm(x, w[p + "post_attention_layernorm.weight"], d["eps"])
    gate = torch.softmax(hn @ w[p + "mlp.router.weight"].T, dim=-1)
    routed = torch.zeros_like(x)
    for i in range(t):
        k = int(gate[i].argmax())
        gu = w[p + f"mlp.experts.{k}.gate_up.weight"]
        half = gu.shape[0] // 2
        routed[i] = gate[i, k] * plain.swiglu(hn[i:i + 1], gu[:half], gu[half:], w[p + f"mlp.experts.{k}.down.weight"])[0]
    x = x + routed
    x, _ = attn_layer(x)
    x, _ = attn_layer(x, kv_from=first_normed)          # reads the keys and values of the first run
    x = plain.rmsnorm(x, w["model.norm.weight"], d["eps"])
    logits = x @ w["model.embed_tokens.weight"].T
    return d["logit_cap"] * torch.tanh(logits / d["logit_cap"]) if "logit_cap" in d else logits


def trace_three_together(requests, tail=6):
    """Three requests, each most of its prompt in a step of its own, then their last ``tail`` tokens
    side by side: steps of three single tokens (which a graph of four rows serves, one row filled in)."""
    rids = [rid for rid, toks in requests.items() if len(toks) > tail][:3]
    steps = [{"step": k, "entries": [{"id": rid, "tokens": requests[rid][:-tail],
                                      "want": list(range(len(requests[rid]) - tail))}], "end": []}
             for k, rid in enumerate(rids)]
    for j in range(tail):
        steps.append({"step": len(steps), "end": rids if j == tail - 1 else [],
                      "entries": [{"id": rid, "tokens": [requests[rid][j - tail]], "want": [0]} for rid in rids]})
    return steps


def run_toy(tmp_path, device, dtype_name, toy=TOY):
    from tinyinfer_b200.engine.replay import TraceSession
    from tinyinfer_b200.config import load_config
    from tinyinfer_b200.weights import load_weights, write_random_model
    folder = write_random_model(tmp_path / "toy", ToyConfig(toy), seed=11, std=0.08)
    assert json.loads((folder / "config.json").read_text())["architectures"] == toy["architectures"]
    arch, cfg = load_config(folder)
    model = arch.model_factory(cfg, torch.float32, torch.device(device))
    load_weights(model, folder)
    needs = model.cache_needs()
    assert needs[1][0] is None and needs[1][1].shape == (48,) and needs[0][0].num_kv_heads == 1
    _, w = plain.read_model_folder(folder, torch.float64)
    requests = helpers.random_requests(dict(vocab_size=97), [40, 9, 70, 33, 2, 50], seed=2)
    want = {rid: toy_plain(w, toks, toy).numpy() for rid, toks in requests.items()}
    replays = 0
    for steps in (helpers.trace_whole(requests), helpers.trace_chunked(requests, seed=4),
                  helpers.trace_mixed(requests, seed=5, max_live=3), trace_three_together(requests)):
        # three state slots for six requests: slots are used again and must start from zero
        session = TraceSession(None, dtype_name, helpers.peak_tokens(steps), page_size=8, model=model,
                               max_live=3, poison_cache=True)
        got = helpers.collect(session, steps)
        assert helpers.first_bad(got, want, 5e-5) is None
        session.runner.manager.check_consistency()
        replays += session.runner.graph_replays
    return replays


TOYS = dict(argvalues=[TOY, TOY_PAIRS, TOY_ON_DEVICE, TOY_FRAMED],
            ids=["stretched", "pairs_from_table", "state_on_device", "framed"])


@pytest.mark.gpu
@pytest.mark.parametrize("toy", **TOYS)
def test_toy_architecture_steps_on_the_gpu(tmp_path, toy):
    replays = run_toy(tmp_path, "cuda:0", "float32", toy)
    # a mixer that reads its state slots on the host keeps the model's steps out of CUDA graphs; with the one
    # that leaves them on the device the steps of single tokens are replayed, three requests in a graph of four rows
    assert (replays > 0) == (toy is TOY_ON_DEVICE)


@pytest.mark.parametrize("toy", **TOYS)
def test_toy_architecture_steps_with_plain_ops(tmp_path, monkeypatch, toy):
    from tinyinfer_b200 import ops
    for name in torch_ops.ALL:
        monkeypatch.setattr(ops, name, getattr(torch_ops, name))
    run_toy(tmp_path, "cpu", "float32", toy)
