"""A whole architecture added from outside the package: a configuration class of its own keys, a spec builder, a
registry entry, a block arrangement and a feed-forward that the package does not have, other tensor names, partial
rotation and no per-head norms. Everything is defined in this file; the model folder is written by the package's
random-weights mode, found by ``config.json``'s ``architectures``, loaded by tensor name and replayed in mixed
batches against a plain computation. It is a toy: no model of anyone's."""
import dataclasses
import json
import os

import numpy as np
import pytest
import torch

import plain_qwen3 as P
import replay_util as RU

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@dataclasses.dataclass(frozen=True)
class ToyConfig:
    dim: int
    n_layers: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    rotary_dim: int
    ffn_dim: int
    vocab: int
    theta: float
    eps: float
    max_len: int

    @classmethod
    def from_dict(cls, raw):
        return cls(**{f.name: raw[f.name] for f in dataclasses.fields(cls)})

    def to_dict(self):
        return {"architectures": ["ToyParallelForCausalLM"], "model_type": "toy_parallel", **dataclasses.asdict(self)}


def _register():
    from llm_rs_b200.config import ArchitectureEntry, register_architecture
    from llm_rs_b200.parts import (Block, FeedForward, LayerSpec, ModelSpec, PartSpec, RunStep, WeightSpec, build,
                                   register)

    @register("block", "toy_parallel", replace=True)
    class ParallelBlock(Block):
        """h += mixer(norm(h)) + feed_forward(norm(h)): one norm, both branches read it."""

        def __init__(self, layer, prefix=""):
            p = layer.prefix
            self.norm = build("norm", layer.mixer_norm, prefix=p)
            self.mixer = build("mixer", layer.mixer, prefix=p + layer.mixer_scope)
            self.feed_forward = build("feed_forward", layer.feed_forward, prefix=p + layer.feed_forward_scope)

        def parts(self):
            return [self.norm, self.mixer, self.feed_forward]

        def weight_specs(self):
            return [s for part in self.parts() for s in part.weight_specs()]

        def bind(self, tensors, runtime):
            for part in self.parts():
                part.bind(tensors, runtime)

        def forward(self, h, pending, ctx, cache):
            x = self.norm.forward(h, pending)
            return h, self.mixer.forward(x, ctx, cache) + self.feed_forward.forward(x, ctx)

    @register("feed_forward", "toy_relu2", replace=True)
    class ReluSquared(FeedForward):
        """down(relu(up(x))^2), float32 arithmetic."""

        def __init__(self, dim, ffn_dim, prefix=""):
            self.dim, self.ffn_dim, self.prefix = dim, ffn_dim, prefix

        def weight_specs(self):
            return [WeightSpec(self.prefix + "w_up.weight", (self.ffn_dim, self.dim)),
                    WeightSpec(self.prefix + "w_down.weight", (self.dim, self.ffn_dim))]

        def bind(self, tensors, runtime):
            self.up, self.down = tensors[self.prefix + "w_up.weight"].float(), tensors[self.prefix + "w_down.weight"].float()

        def forward(self, x, ctx):
            return ((torch.relu(x.float() @ self.up.t()) ** 2) @ self.down.t()).to(x.dtype)

    def build_spec(cfg: ToyConfig) -> ModelSpec:
        norm = lambda name: PartSpec("rmsnorm", {"dim": cfg.dim, "eps": cfg.eps, "name": name})
        layers = []
        for i in range(cfg.n_layers):
            mixer = PartSpec("gqa_attention", {
                "hidden_size": cfg.dim, "n_heads": cfg.n_heads, "n_kv_heads": cfg.n_kv_heads, "head_dim": cfg.head_dim,
                "position": PartSpec("rope_half", {"head_dim": cfg.head_dim, "theta": cfg.theta, "rotary_dim": cfg.rotary_dim}),
                "qk_norm": False, "names": {"q": "wq", "k": "wk", "v": "wv", "o": "wo"}})
            layers.append(LayerSpec(
                prefix=f"layers.{i}.", block=PartSpec("toy_parallel"), mixer=mixer,
                feed_forward=PartSpec("toy_relu2", {"dim": cfg.dim, "ffn_dim": cfg.ffn_dim}),
                mixer_norm=norm("norm.weight"),
                mixer_scope="attention.", feed_forward_scope="feed_forward."))
        return ModelSpec(
            hidden_size=cfg.dim, vocab_size=cfg.vocab, layers=tuple(layers),
            run_order=tuple(RunStep(i) for i in range(cfg.n_layers)),
            embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.dim, "name": "tok_embeddings.weight"}),
            final_norm=norm("norm.weight"),
            lm_head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.dim, "name": "output.weight"}),
            max_positions=cfg.max_len, eos_token_ids=())

    register_architecture(ArchitectureEntry(name="ToyParallelForCausalLM", model_type="toy_parallel",
                                            config_cls=ToyConfig, build_spec=build_spec), replace=True)


def _unregister():
    from llm_rs_b200.config import unregister_architecture
    from llm_rs_b200.parts import unregister
    unregister_architecture("ToyParallelForCausalLM")
    unregister("block", "toy_parallel")
    unregister("feed_forward", "toy_relu2")


def _plain(cfg: ToyConfig, w, toks):
    """The toy architecture on whole sequences in float64, from the plain implementation's parts."""
    T, d, rot = len(toks), cfg.head_dim, cfg.rotary_dim
    h = P.embedding(w["tok_embeddings.weight"], toks)
    ang = P.rope_angles(range(T), rot, cfg.theta, torch.float64)
    def rotate(x):      # the first ``rot`` elements of every head are rotated, the rest pass
        return torch.cat([P.rotate_half(x[..., :rot], ang), x[..., rot:]], dim=-1)
    for i in range(cfg.n_layers):
        p = f"layers.{i}."
        x = P.rms_norm(h, w[p + "norm.weight"], cfg.eps)
        q = rotate(P.linear(x, w[p + "attention.wq.weight"]).reshape(T, cfg.n_heads, d))
        k = rotate(P.linear(x, w[p + "attention.wk.weight"]).reshape(T, cfg.n_kv_heads, d))
        v = P.linear(x, w[p + "attention.wv.weight"]).reshape(T, cfg.n_kv_heads, d)
        a = P.linear(P.attention(q, k, v), w[p + "attention.wo.weight"])
        f = (torch.relu(P.linear(x, w[p + "feed_forward.w_up.weight"])) ** 2) @ w[p + "feed_forward.w_down.weight"].t()
        h = h + a + f
    return P.linear(P.rms_norm(h, w["norm.weight"], cfg.eps), w["output.weight"])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_a_whole_toy_architecture_is_added_from_outside(tmp_path, dtype):
    from llm_rs_b200.config import architecture_names, load_config
    from llm_rs_b200.engine import Engine, EngineConfig, ModelRunner
    from llm_rs_b200.sampling import SamplingParams
    from llm_rs_b200.weights import write_random_model
    _register()
    try:
        assert "ToyParallelForCausalLM" in architecture_names()
        cfg = ToyConfig(dim=88, n_layers=3, n_heads=6, n_kv_heads=2, head_dim=16, rotary_dim=8, ffn_dim=120, vocab=211,
                        theta=5000.0, eps=1e-5, max_len=400)
        path = write_random_model(str(tmp_path / "toy"), cfg, seed=21, sigma=0.06, norm_jitter=0.1)
        raw = json.load(open(os.path.join(path, "config.json")))
        assert raw["architectures"] == ["ToyParallelForCausalLM"] and raw["rotary_dim"] == 8
        entry, loaded = load_config(path)
        assert entry.config_cls is ToyConfig and loaded == cfg
        _, w = P.load_model_dir(path)
        assert "layers.2.attention.wq.weight" in w and "layers.0.feed_forward.w_up.weight" in w and "output.weight" in w
        assert not any("q_norm" in n or "mlp" in n or "unused" in n for n in w)
        rng = np.random.default_rng(33)
        reqs = {f"r{i}": rng.integers(0, cfg.vocab, n).tolist() for i, n in enumerate((60, 17, 130, 5, 75))}
        ref = {r: _plain(cfg, w, t).numpy() for r, t in reqs.items()}
        steps = RU.mixed(reqs, seed=6)
        runner = ModelRunner.from_model_dir(path, dtype=dtype, max_tokens=RU.live_token_peak(steps), page_size=16,
                                            max_requests=4)
        runner.use_graphs = True
        got = RU.run_steps(runner, steps)
        worst, where, n = RU.max_diff(got, ref)
        assert n == sum(len(t) for t in reqs.values())
        tol = 1e-4 if dtype == torch.float32 else 0.02 * max(float(np.abs(r).max()) for r in ref.values())
        assert worst <= tol, (worst, where)
        # And through the engine: greedy tokens are the plain computation's own.
        engine = Engine(EngineConfig(model_path=path, block_pool_size=32, dtype="float32", max_requests=4))
        out = engine.generate([reqs["r1"]], SamplingParams(temperature=0.0, max_new_tokens=5))[0]
        seq = list(reqs["r1"])
        for tok in out:
            assert tok == int(_plain(cfg, w, seq)[-1].argmax())
            seq.append(tok)
    finally:
        _unregister()
