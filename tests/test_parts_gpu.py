"""Each part alone against its plain function, and the generality of the assembly: a toy
mixer with state of its own and a toy architecture whose schedule runs a layer twice and lets
a layer read another layer's cache, all defined here and registered through the public
calls, without touching the package."""
from dataclasses import dataclass
from typing import ClassVar

import pytest
import torch

import plain_qwen2 as plain
import replay_util as ru

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def make_ctx(entries, groups, page_size, num_pages, dtype, tile_tokens=(), state_needs=(), harness=None):
    from dispec_b200.cache import CacheManager
    from dispec_b200.cache.storage import CacheStorage, StateStorage
    from dispec_b200.engine.batch import HostStaging, build_context
    if harness is None:
        cache = CacheManager(groups, page_size, num_pages, 8)
        harness = dict(cache=cache, storage=CacheStorage(groups, page_size, [num_pages] * len(groups), dtype, DEV, poison=True),
                       states=StateStorage(list(state_needs), 8, DEV), staging=HostStaging(DEV))
    cache = harness["cache"]
    for e in entries:
        if not cache.has(e.req_id):
            cache.admit(e.req_id)
        cache.extend(e.req_id, e.start + len(e.tokens))
    ctx, _ = build_context(entries, cache, harness["storage"], harness["states"], harness["staging"], dtype,
                           torch.device(DEV), list(tile_tokens), 1 << 30)
    return ctx, harness


def _tile_sizes(mixer):
    want = mixer.tokens_per_attention_tile()
    if not want:
        return []
    return list(want) if isinstance(want, (tuple, list)) else [want]


def commit(harness, entries):
    for e in entries:
        harness["cache"].commit(e.req_id, e.start + len(e.tokens))


def rnd(shape, seed, scale=1.0):
    return torch.randn(shape, generator=torch.Generator().manual_seed(seed)) * scale


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rms_norm_part(dtype):
    from dispec_b200.engine import SeqEntry
    from dispec_b200.parts.norms import RMSNorm
    norm = RMSNorm(hidden_size=72, eps=1e-5)
    assert norm.tensor_specs()["weight"].shape == (72,)
    w = (1 + rnd((72,), 1, 0.1)).to(dtype)
    norm.load({"weight": w.to(DEV)})
    x, d = rnd((6, 72), 2).to(dtype), rnd((6, 72), 3).to(dtype)
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    y = norm.forward(None, x.to(DEV))
    torch.testing.assert_close(y.float().cpu(), plain.rms_norm(x.float(), w.float(), 1e-5), atol=tol, rtol=tol)
    resid = x.to(DEV).clone()
    y2 = norm.forward_add(None, resid, d.to(DEV))
    s = (x.float() + d.float()).to(dtype)
    assert torch.equal(resid.cpu(), s)
    torch.testing.assert_close(y2.float().cpu(), plain.rms_norm(s.float(), w.float(), 1e-5), atol=tol, rtol=tol)


def test_rotary_part_matches_the_plain_tables():
    from dispec_b200.parts.rotary import RotaryEncoding
    pe = RotaryEncoding(head_dim=48, theta=50000.0)
    pe.prepare(DEV)
    pos = torch.tensor([0, 1, 77, 4000])
    cos, sin = plain.rope_tables(pos, 48, 50000.0)
    ang = pos.float()[:, None] * pe.inv_freq.cpu()[None]
    assert torch.equal(torch.cat([ang, ang], -1).cos(), cos)
    assert pe.rotation().rotary_dim == 48 and pe.rotation().inv_freq is pe.inv_freq and pe.score_scale() == 1.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu_part(dtype):
    from dispec_b200.parts.swiglu import SwiGLUFeedForward
    ff = SwiGLUFeedForward(hidden_size=72, intermediate_size=200)
    wg, wu, wd = rnd((200, 72), 4, 0.2).to(dtype), rnd((200, 72), 5, 0.2).to(dtype), rnd((72, 200), 6, 0.2).to(dtype)
    ff.load({"gate_proj.weight": wg.to(DEV), "up_proj.weight": wu.to(DEV), "down_proj.weight": wd.to(DEV)})
    x = rnd((5, 72), 7).to(dtype)
    y = ff.forward(None, x.to(DEV)).float().cpu()
    ref = plain.swiglu_mlp(x.float(), wg.float(), wu.float(), wd.float())
    tol = 2e-5 if dtype == torch.float32 else 5e-2
    torch.testing.assert_close(y, ref, atol=tol, rtol=tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_and_head_parts(dtype):
    from dispec_b200.engine import SeqEntry
    from dispec_b200.parts.embedding import LinearHead, TokenEmbedding
    emb, head = TokenEmbedding(101, 40), LinearHead(101, 40)
    table = rnd((101, 40), 8).to(dtype).to(DEV)
    emb.load({"weight": table})
    head.load({"weight": table})
    ctx, _ = make_ctx([SeqEntry("s", [100, 0, 7], 0, [])], [], 4, 4, dtype)
    x = emb.forward(ctx)
    assert torch.equal(x, table[[100, 0, 7]])
    logits = head.forward(ctx, x)
    assert logits.dtype == torch.float32
    torch.testing.assert_close(logits.cpu(), x.float().cpu() @ table.float().cpu().T,
                               atol=1e-4 if dtype == torch.float32 else 2e-2, rtol=1e-3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [0, 9])
def test_attention_part_in_two_portions(dtype, window):
    from dispec_b200.cache import CacheGroupSpec
    from dispec_b200.engine import SeqEntry
    from dispec_b200.parts.attention import GQAAttention
    from dispec_b200.parts.rotary import RotaryEncoding
    H, KVH, D, hidden = 6, 2, 32, 72
    pe = RotaryEncoding(D, 20000.0)
    pe.prepare(DEV)
    mixer = GQAAttention(hidden, H, KVH, D, qkv_bias=True, position_encoding=pe, window=window)
    specs = mixer.tensor_specs()
    cpu = {n: rnd(s.shape, 10 + i, 0.15).to(dtype) for i, (n, s) in enumerate(specs.items())}
    mixer.load({n: t.to(DEV) for n, t in cpu.items()})
    assert mixer.cache_need().window == window and [t.name for t in mixer.cache_need().tensors] == ["key", "value"]
    T = 29
    x = rnd((T, hidden), 40).to(dtype)
    groups = [CacheGroupSpec.key_value(KVH, D, window, 1)]
    tiles = _tile_sizes(mixer)
    from dispec_b200.models.model import CachePlacement
    out, harness, pos = [], None, 0
    for n in (18, 11):
        e = [SeqEntry("s", list(range(n)), pos, [])]
        ctx, harness = make_ctx(e, groups, 8, 6, dtype, tiles, harness=harness)
        out.append(mixer.forward(ctx, x[pos:pos + n].to(DEV), ctx.cache_view(CachePlacement(0, 0), True), None))
        commit(harness, e)
        pos += n
    got = torch.cat(out).float().cpu()
    f = {n: t.float() for n, t in cpu.items()}
    q, k, v = plain.qkv_projection(x.float(), f["q_proj.weight"], f["q_proj.bias"], f["k_proj.weight"],
                                   f["k_proj.bias"], f["v_proj.weight"], f["v_proj.bias"], H, KVH, D)
    cos, sin = plain.rope_tables(torch.arange(T), D, 20000.0)
    o = plain.causal_attention(plain.apply_rope(q, cos, sin), plain.apply_rope(k, cos, sin), v, window)
    ref = o.reshape(T, -1) @ f["o_proj.weight"].T
    tol = 2e-5 if dtype == torch.float32 else 5e-2
    torch.testing.assert_close(got, ref, atol=tol, rtol=tol)


BLOCK_SIZES = dict(H=4, KVH=2, D=32, hidden=96, inter=208, eps=1e-5, theta=30000.0)


def _make_block(dtype, seed, prefix, weights):
    """A pre-norm block of the package's own parts with random weights (also put into ``weights``
    under the plain implementation's names)."""
    from dispec_b200.parts.attention import GQAAttention
    from dispec_b200.parts.block import PreNormBlock
    from dispec_b200.parts.norms import RMSNorm
    from dispec_b200.parts.rotary import RotaryEncoding
    from dispec_b200.parts.swiglu import SwiGLUFeedForward
    z = BLOCK_SIZES
    pe = RotaryEncoding(z["D"], z["theta"])
    pe.prepare(DEV)
    parts = dict(n1=RMSNorm(z["hidden"], z["eps"]), n2=RMSNorm(z["hidden"], z["eps"]),
                 mixer=GQAAttention(z["hidden"], z["H"], z["KVH"], z["D"], True, pe),
                 ffn=SwiGLUFeedForward(z["hidden"], z["inter"]))
    names = {"n1": {"weight": "input_layernorm.weight"}, "n2": {"weight": "post_attention_layernorm.weight"},
             "mixer": {f"{n}_proj.{k}": f"self_attn.{n}_proj.{k}" for n in "qkv" for k in ("weight", "bias")}
             | {"o_proj.weight": "self_attn.o_proj.weight"},
             "ffn": {f"{n}_proj.weight": f"mlp.{n}_proj.weight" for n in ("gate", "up", "down")}}
    for key, part in parts.items():
        local = {}
        for n, spec in part.tensor_specs().items():
            t = rnd(spec.shape, seed, 0.12)
            seed += 1
            if spec.init == "one_plus_normal":
                t = t + 1.0
            t = t.to(dtype)
            weights[prefix + names[key][n]] = t.float()
            local[n] = t.to(DEV)
        part.load(local)
    return PreNormBlock(parts["n1"], parts["mixer"], parts["n2"], parts["ffn"]), parts


class NormKernelOnly:
    """A norm that offers the two methods every norm has and nothing else: the block then runs it
    as a kernel of its own and lets the products add the residual stream."""

    def __init__(self, norm):
        self._norm = norm

    def forward(self, ctx, x, rows=None):
        return self._norm.forward(ctx, x, rows=rows)

    def forward_add(self, ctx, residual, delta, rows=None):
        return self._norm.forward_add(ctx, residual, delta, rows=rows)


@pytest.mark.parametrize("norms_in_products", [True, False])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_pre_norm_block_alone(dtype, norms_in_products):
    """The arrangement of a layer (two norms, mixer, feed-forward, residual sums) against the
    plain layer function, a sequence in two portions; with norms that can be handed to the
    products after them and with norms that cannot."""
    from dispec_b200.cache import CacheGroupSpec
    from dispec_b200.engine import SeqEntry
    from dispec_b200.models.model import CachePlacement
    from dispec_b200.parts.block import PreNormBlock
    z = BLOCK_SIZES
    weights = {}
    block, parts = _make_block(dtype, 200, "L.", weights)
    if not norms_in_products:
        block = PreNormBlock(NormKernelOnly(parts["n1"]), parts["mixer"], NormKernelOnly(parts["n2"]), parts["ffn"])
        assert block.first_norm_after_product() is None
    T = 23
    x = rnd((T, z["hidden"]), 300).to(dtype)
    groups = [CacheGroupSpec.key_value(z["KVH"], z["D"], 0, 1)]
    out, harness, pos = [], None, 0
    for n in (9, 14):
        e = [SeqEntry("s", list(range(n)), pos, [])]
        ctx, harness = make_ctx(e, groups, 8, 6, dtype, _tile_sizes(parts["mixer"]), harness=harness)
        xs, pending = block.forward(ctx, x[pos:pos + n].to(DEV).clone(), None, ctx.cache_view(CachePlacement(0, 0), True), None)
        out.append(xs if pending is None else xs + pending)
        commit(harness, e)
        pos += n
    got = torch.cat(out).float().cpu()
    c = dict(eps=z["eps"], heads=z["H"], kv_heads=z["KVH"], head_dim=z["D"])
    cos, sin = plain.rope_tables(torch.arange(T), z["D"], z["theta"])
    ref = plain.decoder_layer(x.float(), weights, "L.", c, cos, sin, 0)
    tol = 3e-5 if dtype == torch.float32 else 6e-2
    torch.testing.assert_close(got, ref, atol=tol, rtol=tol)


@pytest.mark.parametrize("dtype,rows", [(torch.bfloat16, 11), (torch.bfloat16, 70), (torch.float32, 11)])
def test_pre_norm_blocks_hand_their_norms_to_the_products(dtype, rows):
    """Two blocks in a row, the first told which norm reads its result: it hands that norm on,
    still to be applied; with few rows in bfloat16 the scaled copy is there and the norms run
    inside the products, otherwise the second block runs the norm kernel.  Either way the result
    is the plain two layers."""
    from dispec_b200.cache import CacheGroupSpec
    from dispec_b200.engine import SeqEntry
    from dispec_b200.models.model import CachePlacement
    from dispec_b200.ops.gemm import NORM_SPLIT_MAX_ROWS, NormedRows
    z = BLOCK_SIZES
    weights = {}
    first, parts1 = _make_block(dtype, 400, "A.", weights)
    second, parts2 = _make_block(dtype, 500, "B.", weights)
    x = rnd((rows, z["hidden"]), 600).to(dtype)
    groups = [CacheGroupSpec.key_value(z["KVH"], z["D"], 0, 2)]
    e = [SeqEntry("s", list(range(rows)), 0, [])]
    ctx, harness = make_ctx(e, groups, 8, 2 * (rows // 8 + 2), dtype, _tile_sizes(parts1["mixer"]))
    offer = second.first_norm_after_product()
    assert offer is not None and offer[0] is parts2["n1"].weight
    h, pending = first.forward(ctx, x.to(DEV).clone(), None, ctx.cache_view(CachePlacement(0, 0), True), None,
                               then_norm=offer)
    assert isinstance(pending, NormedRows) and pending.source is h and pending.weight is parts2["n1"].weight
    if dtype == torch.bfloat16 and rows <= NORM_SPLIT_MAX_ROWS:
        assert torch.equal(pending.scaled, (h.float() * parts2["n1"].weight.float()).to(dtype))
    else:
        assert pending.scaled is None
    out, last = second.forward(ctx, h, pending, ctx.cache_view(CachePlacement(0, 1), True), None)
    assert last is None
    c = dict(eps=z["eps"], heads=z["H"], kv_heads=z["KVH"], head_dim=z["D"])
    cos, sin = plain.rope_tables(torch.arange(rows), z["D"], z["theta"])
    ref = plain.decoder_layer(plain.decoder_layer(x.float(), weights, "A.", c, cos, sin, 0), weights, "B.", c, cos, sin, 0)
    tol = 6e-5 if dtype == torch.float32 else 1e-1
    torch.testing.assert_close(out.float().cpu(), ref, atol=tol, rtol=tol)


# ------------------------------------------------------------------- toy parts and models

def register_toys():
    """A mixer with fixed-size state of its own (a per-channel decaying sum), and two toy
    architectures.  Registered once per process through the public calls."""
    from dispec_b200 import register_architecture, register_part
    from dispec_b200.config.model_config import ModelConfig
    from dispec_b200.models.spec import LayerCall, ModelSpec
    from dispec_b200.parts.base import Mixer, PartSpec, StateNeed, TensorSpec
    from dispec_b200.registry import architectures

    if "ToyStateForCausalLM" in architectures():
        return

    @register_part("mixer", "toy_decay")
    class DecayMixer(Mixer):
        """s_t = sigmoid(a) * s_{t-1} + x_t W_in^T ;  y_t = s_t W_out^T.  The state s lives in
        the request's state slot and is carried across portions and steps."""

        def __init__(self, hidden_size, state_size):
            self.hidden_size, self.state_size = hidden_size, state_size

        def tensor_specs(self):
            return {"in.weight": TensorSpec((self.state_size, self.hidden_size)),
                    "out.weight": TensorSpec((self.hidden_size, self.state_size)),
                    "decay": TensorSpec((self.state_size,), dtype="float32")}

        def load(self, tensors):
            self.w_in, self.w_out, self.decay = tensors["in.weight"], tensors["out.weight"], tensors["decay"]
            assert self.decay.dtype == torch.float32  # stays 32-bit in every mode

        def state_need(self):
            return StateNeed((self.state_size,), "float32")

        def forward(self, ctx, x, cache, state):
            assert cache is None
            u = x.float() @ self.w_in.float().T
            y = torch.empty_like(u)
            a = torch.sigmoid(self.decay)
            for s in range(ctx.num_seqs):
                slot = ctx.host_state_slot[s]
                st = state.buffer[slot]
                for t in range(ctx.host_q_start[s], ctx.host_q_start[s + 1]):
                    st = a * st + u[t]
                    y[t] = st
                state.buffer[slot] = st
            return (y @ self.w_out.float().T).to(x.dtype)

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        architecture: ClassVar[str] = "ToyStateForCausalLM"
        vocab_size: int = 0
        hidden_size: int = 0
        state_size: int = 0
        intermediate_size: int = 0
        num_layers: int = 0
        eps: float = 0.0

        @classmethod
        def from_dict(cls, d):
            return cls(**{k: d[k] for k in ("vocab_size", "hidden_size", "state_size",
                                            "intermediate_size", "num_layers", "eps")})

        def to_dict(self):
            return dict(architectures=[self.architecture], **{k: getattr(self, k) for k in (
                "vocab_size", "hidden_size", "state_size", "intermediate_size", "num_layers", "eps")})

    def build_toy(cfg):
        h = cfg.hidden_size
        layers = []
        for i in range(cfg.num_layers):
            p = f"layers.{i}."
            norm = lambda n: PartSpec("norm", "rms_norm", {"hidden_size": h, "eps": cfg.eps}, {"weight": p + n})
            mixer = PartSpec("mixer", "toy_decay", {"hidden_size": h, "state_size": cfg.state_size},
                             {"in.weight": p + "mix.in", "out.weight": p + "mix.out", "decay": p + "mix.decay"})
            ffn = PartSpec("feed_forward", "swiglu", {"hidden_size": h, "intermediate_size": cfg.intermediate_size},
                           {f"{n}_proj.weight": p + "ffn." + n for n in ("gate", "up", "down")})
            layers.append(PartSpec("block", "pre_norm", {"mixer_norm": norm("n1"), "mixer": mixer,
                                                         "ffn_norm": norm("n2"), "feed_forward": ffn}))
        return ModelSpec("ToyStateForCausalLM",
                         PartSpec("embedding", "token_embedding", {"vocab_size": cfg.vocab_size, "hidden_size": h}, {"weight": "emb"}),
                         layers,
                         PartSpec("norm", "rms_norm", {"hidden_size": h, "eps": cfg.eps}, {"weight": "final"}),
                         PartSpec("head", "linear_head", {"vocab_size": cfg.vocab_size, "hidden_size": h}, {"weight": "emb"}),
                         vocab_size=cfg.vocab_size, max_position=4096)

    register_architecture("ToyStateForCausalLM", ToyConfig, build_toy)

    # a Qwen2-shaped toy whose schedule runs layer 0 twice and lets the last call of layer 1
    # read the cache its first call wrote
    from dispec_b200.config import Qwen2Config
    from dispec_b200.models.qwen2 import build_qwen2

    @dataclass(frozen=True)
    class LoopConfig(Qwen2Config):
        architecture: ClassVar[str] = "ToyLoopForCausalLM"

    def build_loop(cfg):
        spec = build_qwen2(cfg)
        spec.architecture = "ToyLoopForCausalLM"
        spec.schedule = [LayerCall(0, 0, True), LayerCall(1, 1, True), LayerCall(0, 2, True),
                         LayerCall(1, 1, False)]
        return spec

    register_architecture("ToyLoopForCausalLM", LoopConfig, build_loop)


def plain_toy_state(weights, cfg, ids):
    x = weights["emb"][torch.as_tensor(ids)]
    for i in range(cfg["num_layers"]):
        p = f"layers.{i}."
        h = plain.rms_norm(x, weights[p + "n1"], cfg["eps"])
        u = h @ weights[p + "mix.in"].T
        a = torch.sigmoid(weights[p + "mix.decay"])
        st = torch.zeros(cfg["state_size"])
        ys = []
        for t in range(len(ids)):
            st = a * st + u[t]
            ys.append(st)
        x = x + torch.stack(ys) @ weights[p + "mix.out"].T
        h = plain.rms_norm(x, weights[p + "n2"], cfg["eps"])
        x = x + plain.swiglu_mlp(h, weights[p + "ffn.gate"], weights[p + "ffn.up"], weights[p + "ffn.down"])
    return plain.rms_norm(x, weights["final"], cfg["eps"]) @ weights["emb"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_mixer_with_state_is_registered_built_and_stepped(tmp_path, dtype):
    from safetensors.torch import load_file
    from dispec_b200 import load_model, load_model_config, write_random_model
    from dispec_b200.engine import ModelRunner, SeqEntry
    register_toys()
    cfg_dict = dict(architectures=["ToyStateForCausalLM"], vocab_size=90, hidden_size=48, state_size=40,
                    intermediate_size=64, num_layers=2, eps=1e-5)
    cfg = load_model_config(cfg_dict)
    write_random_model(cfg, str(tmp_path), seed=3, std=0.2, dtype="bfloat16")
    weights = {k: v.float() for k, v in load_file(str(tmp_path / "model.safetensors")).items()}
    model = load_model(str(tmp_path), dtype, DEV)
    assert model.cache_groups == [] and len(model.state_needs) == 2
    assert model.layers[0].mixer.decay.dtype == torch.float32
    runner = ModelRunner(model, page_size=16, num_pages=4, max_num_seqs=3)
    a, b = ru.random_ids(23, 90, 1), ru.random_ids(11, 90, 2)
    ref_a, ref_b = plain_toy_state(weights, cfg_dict, a), plain_toy_state(weights, cfg_dict, b)
    runner.admit("a")
    runner.admit("b")
    got_a, got_b = [], []
    # a in portions and single tokens, b beside it, cut anywhere
    got_a.append(runner.step([SeqEntry("a", a[:9], 0, list(range(9)))]))
    l = runner.step([SeqEntry("a", a[9:10], 9, [0]), SeqEntry("b", b[:6], 0, list(range(6)))])
    got_a.append(l[:1]); got_b.append(l[1:])
    l = runner.step([SeqEntry("b", b[6:7], 6, [0]), SeqEntry("a", a[10:23], 10, list(range(13)))])
    got_b.append(l[:1]); got_a.append(l[1:])
    got_b.append(runner.step([SeqEntry("b", b[7:], 7, list(range(4)))]))
    tol = 1e-4 if dtype == "float32" else 0.05
    scale = max(1.0, ref_a.abs().max().item())
    assert (torch.cat(got_a).cpu() - ref_a).abs().max().item() < tol * scale
    assert (torch.cat(got_b).cpu() - ref_b).abs().max().item() < tol * scale
    # a state slot is zeroed when it is handed to the next request
    runner.release("a")
    runner.admit("c")
    again = runner.step([SeqEntry("c", a, 0, list(range(len(a))))])
    assert (again.cpu() - ref_a).abs().max().item() < tol * scale


def plain_loop(weights, config, ids):
    c = plain.read_config(config)
    w = weights
    T = len(ids)
    cos, sin = plain.rope_tables(torch.arange(T), c["head_dim"], c["theta"])
    x = plain.embed(w["model.embed_tokens.weight"], torch.as_tensor(ids))
    x = plain.decoder_layer(x, w, "model.layers.0.", c, cos, sin, 0)
    # layer 1, first call: remember its rotated keys and its values
    p = "model.layers.1."
    a = p + "self_attn."
    kept = {}

    def layer1(x, reuse):
        h = plain.rms_norm(x, w[p + "input_layernorm.weight"], c["eps"])
        q, k, v = plain.qkv_projection(h, w[a + "q_proj.weight"], w[a + "q_proj.bias"], w[a + "k_proj.weight"],
                                       w[a + "k_proj.bias"], w[a + "v_proj.weight"], w[a + "v_proj.bias"],
                                       c["heads"], c["kv_heads"], c["head_dim"])
        q, k = plain.apply_rope(q, cos, sin), plain.apply_rope(k, cos, sin)
        if reuse:
            k, v = kept["k"], kept["v"]
        else:
            kept["k"], kept["v"] = k, v
        o = plain.causal_attention(q, k, v)
        x = x + o.reshape(T, -1) @ w[a + "o_proj.weight"].T
        h = plain.rms_norm(x, w[p + "post_attention_layernorm.weight"], c["eps"])
        return x + plain.swiglu_mlp(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                                    w[p + "mlp.down_proj.weight"])

    x = layer1(x, False)
    x = plain.decoder_layer(x, w, "model.layers.0.", c, cos, sin, 0)
    x = layer1(x, True)
    x = plain.rms_norm(x, w["model.norm.weight"], c["eps"])
    return x @ w["lm_head.weight"].T


def test_schedule_runs_a_layer_twice_and_shares_a_cache(tmp_path):
    import json
    from safetensors.torch import load_file
    from dispec_b200 import load_model, load_model_config, write_random_model
    from dispec_b200.engine import ModelRunner, SeqEntry
    register_toys()
    d = dict(ru.CONFIG_B, architectures=["ToyLoopForCausalLM"], num_hidden_layers=2)
    cfg = load_model_config(d)
    write_random_model(cfg, str(tmp_path), seed=4, std=0.08, dtype="bfloat16")
    cfg_json = json.load(open(tmp_path / "config.json"))
    weights = {k: v.float() for k, v in load_file(str(tmp_path / "model.safetensors")).items()}
    model = load_model(str(tmp_path), "float32", DEV)
    assert len(model.schedule) == 4 and model.cache_groups[0].num_slots == 3
    runner = ModelRunner(model, page_size=8, num_pages=8, max_num_seqs=2, poison=True)
    ids = ru.random_ids(37, d["vocab_size"], 5)
    ref = plain_loop(weights, cfg_json, ids)
    runner.admit("s")
    out, pos = [], 0
    for n in (14, 2, 1, 1, 19):
        out.append(runner.step([SeqEntry("s", ids[pos:pos + n], pos, list(range(n)))]))
        pos += n
    assert (torch.cat(out).cpu() - ref).abs().max().item() < 1e-4


# ------------------------------------------------ a feed-forward with routing, another position encoding

def register_routed_toy():
    """Two more toy parts, registered from here through the public calls: a feed-forward that
    routes every token to one of its experts (32-bit router), and a rotary encoding with
    slowed-down frequencies over half of the head.  A toy architecture uses them in its odd
    layers and the package's own dense feed-forward and rotary encoding in its even ones."""
    from dispec_b200 import register_architecture, register_part
    from dispec_b200.config.model_config import ModelConfig
    from dispec_b200.models.spec import LayerCall, ModelSpec
    from dispec_b200.parts.base import FeedForward, PartSpec, PositionEncoding, Rotation, TensorSpec
    from dispec_b200.registry import architectures

    if "ToyRoutedForCausalLM" in architectures():
        return

    @register_part("feed_forward", "toy_top1_experts")
    class Top1Experts(FeedForward):
        """p = softmax(h Wr^T) in 32-bit; e = argmax p; y = p_e * down_e(silu(gate_e h) * up_e h)."""

        def __init__(self, hidden_size, intermediate_size, num_experts):
            self.h, self.i, self.e = hidden_size, intermediate_size, num_experts

        def tensor_specs(self):
            return {"router.weight": TensorSpec((self.e, self.h), dtype="float32"),
                    "gate.weight": TensorSpec((self.e, self.i, self.h)),
                    "up.weight": TensorSpec((self.e, self.i, self.h)),
                    "down.weight": TensorSpec((self.e, self.h, self.i))}

        def load(self, tensors):
            self.router, self.gate = tensors["router.weight"], tensors["gate.weight"]
            self.up, self.down = tensors["up.weight"], tensors["down.weight"]
            assert self.router.dtype == torch.float32

        def forward(self, ctx, x):
            from dispec_b200 import ops
            probs = torch.softmax(x.float() @ self.router.T, dim=-1)
            top_p, top_e = probs.max(dim=-1)
            out = torch.zeros_like(x)
            for e in range(self.e):  # the package's own products, expert by expert
                rows = (top_e == e).nonzero().flatten()
                if rows.numel() == 0:
                    continue
                h = x.index_select(0, rows)
                act = ops.swiglu(ops.linear(h, torch.cat([self.gate[e], self.up[e]]).contiguous()))
                y = ops.linear(act, self.down[e].contiguous()).float() * top_p[rows, None]
                out.index_copy_(0, rows, y.to(x.dtype))
            return out

    @register_part("position_encoding", "toy_slow_half_rotary")
    class SlowHalfRotary(PositionEncoding):
        """Rotates the first half of each head with frequencies divided by ``factor`` and puts a
        factor of its own on the attention scores (``SCORE_SCALE``)."""
        SCORE_SCALE = 1.3

        def __init__(self, head_dim, theta, factor):
            self.rotary_dim = head_dim // 2
            self.theta, self.factor = float(theta), float(factor)
            self.inv_freq = None

        def prepare(self, device):
            exponent = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32) / self.rotary_dim
            self.inv_freq = (1.0 / (self.theta ** exponent) / self.factor).to(torch.float32).to(device)

        def rotation(self):
            return Rotation(self.inv_freq, self.rotary_dim)

        def score_scale(self):
            return self.SCORE_SCALE

    @dataclass(frozen=True)
    class RoutedConfig(ModelConfig):
        architecture: ClassVar[str] = "ToyRoutedForCausalLM"
        vocab_size: int = 0
        hidden_size: int = 0
        heads: int = 0
        kv_heads: int = 0
        head_dim: int = 0
        intermediate_size: int = 0
        num_experts: int = 0
        num_layers: int = 0
        eps: float = 0.0
        theta: float = 0.0
        factor: float = 1.0

        KEYS: ClassVar[tuple] = ("vocab_size", "hidden_size", "heads", "kv_heads", "head_dim", "intermediate_size",
                                 "num_experts", "num_layers", "eps", "theta", "factor")

        @classmethod
        def from_dict(cls, d):
            return cls(**{k: d[k] for k in cls.KEYS})

        def to_dict(self):
            return dict(architectures=[self.architecture], **{k: getattr(self, k) for k in self.KEYS})

    def build(cfg):
        h = cfg.hidden_size
        layers = []
        for i in range(cfg.num_layers):
            p = f"layers.{i}."
            odd = i % 2 == 1
            norm = lambda n: PartSpec("norm", "rms_norm", {"hidden_size": h, "eps": cfg.eps}, {"weight": p + n})
            pe = (PartSpec("position_encoding", "toy_slow_half_rotary",
                           {"head_dim": cfg.head_dim, "theta": cfg.theta, "factor": cfg.factor}) if odd else
                  PartSpec("position_encoding", "rotary", {"head_dim": cfg.head_dim, "theta": cfg.theta}))
            mixer = PartSpec("mixer", "gqa_attention",
                             {"hidden_size": h, "num_heads": cfg.heads, "num_kv_heads": cfg.kv_heads,
                              "head_dim": cfg.head_dim, "qkv_bias": False, "position_encoding": pe, "window": 0},
                             {f"{n}_proj.weight": f"{p}attn.{n}" for n in "qkvo"})
            if odd:
                ffn = PartSpec("feed_forward", "toy_top1_experts",
                               {"hidden_size": h, "intermediate_size": cfg.intermediate_size, "num_experts": cfg.num_experts},
                               {f"{n}.weight": f"{p}moe.{n}" for n in ("router", "gate", "up", "down")})
            else:
                ffn = PartSpec("feed_forward", "swiglu", {"hidden_size": h, "intermediate_size": cfg.intermediate_size},
                               {f"{n}_proj.weight": f"{p}ffn.{n}" for n in ("gate", "up", "down")})
            layers.append(PartSpec("block", "pre_norm", {"mixer_norm": norm("n1"), "mixer": mixer,
                                                         "ffn_norm": norm("n2"), "feed_forward": ffn}))
        return ModelSpec("ToyRoutedForCausalLM",
                         PartSpec("embedding", "token_embedding", {"vocab_size": cfg.vocab_size, "hidden_size": h}, {"weight": "emb"}),
                         layers,
                         PartSpec("norm", "rms_norm", {"hidden_size": h, "eps": cfg.eps}, {"weight": "final"}),
                         PartSpec("head", "linear_head", {"vocab_size": cfg.vocab_size, "hidden_size": h}, {"weight": "head"}),
                         schedule=[LayerCall(i, i, True) for i in range(cfg.num_layers)],
                         vocab_size=cfg.vocab_size, max_position=4096)

    register_architecture("ToyRoutedForCausalLM", RoutedConfig, build)


def plain_routed(weights, cfg, ids):
    T = len(ids)
    H, KVH, D = cfg["heads"], cfg["kv_heads"], cfg["head_dim"]
    x = weights["emb"][torch.as_tensor(ids)]
    pos = torch.arange(T, dtype=torch.float32)
    for i in range(cfg["num_layers"]):
        p = f"layers.{i}."
        odd = i % 2 == 1
        h = plain.rms_norm(x, weights[p + "n1"], cfg["eps"])
        q = (h @ weights[p + "attn.q"].T).view(T, H, D)
        k = (h @ weights[p + "attn.k"].T).view(T, KVH, D)
        v = (h @ weights[p + "attn.v"].T).view(T, KVH, D)
        rot = D // 2 if odd else D
        inv = 1.0 / (cfg["theta"] ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))
        if odd:
            inv = inv / cfg["factor"]
        ang = pos[:, None] * inv[None, :]
        cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]

        def rotate(t):
            lo, hi, rest = t[..., :rot // 2], t[..., rot // 2:rot], t[..., rot:]
            return torch.cat([lo * cos - hi * sin, hi * cos + lo * sin, rest], dim=-1)

        # the toy encoding of the odd layers scales the scores by 1.3 (folded into q here)
        o = plain.causal_attention(rotate(q) * (1.3 if odd else 1.0), rotate(k), v)
        x = x + o.reshape(T, -1) @ weights[p + "attn.o"].T
        h = plain.rms_norm(x, weights[p + "n2"], cfg["eps"])
        if odd:
            probs = torch.softmax(h @ weights[p + "moe.router"].T, dim=-1)
            top_p, top_e = probs.max(dim=-1)
            y = torch.stack([top_p[t] * plain.swiglu_mlp(h[t:t + 1], weights[p + "moe.gate"][top_e[t]],
                                                         weights[p + "moe.up"][top_e[t]],
                                                         weights[p + "moe.down"][top_e[t]])[0] for t in range(T)])
            x = x + y
        else:
            x = x + plain.swiglu_mlp(h, weights[p + "ffn.gate"], weights[p + "ffn.up"], weights[p + "ffn.down"])
    return plain.rms_norm(x, weights["final"], cfg["eps"]) @ weights["head"].T


def test_toy_routed_feed_forward_and_toy_position_encoding_in_alternate_layers(tmp_path):
    """Registered from the test, built from a config, loaded from the random-weights folder and
    stepped through the package's own step function and cache, without a change to the package."""
    from safetensors.torch import load_file
    from dispec_b200 import load_model, load_model_config, write_random_model
    from dispec_b200.engine import ModelRunner, SeqEntry
    register_routed_toy()
    cfg_dict = dict(architectures=["ToyRoutedForCausalLM"], vocab_size=77, hidden_size=40, heads=4, kv_heads=2,
                    head_dim=16, intermediate_size=48, num_experts=3, num_layers=4, eps=1e-5, theta=5000.0, factor=4.0)
    cfg = load_model_config(cfg_dict)
    write_random_model(cfg, str(tmp_path), seed=6, std=0.15, dtype="bfloat16")
    weights = {k: v.float() for k, v in load_file(str(tmp_path / "model.safetensors")).items()}
    model = load_model(str(tmp_path), "float32", DEV)
    assert [type(l.feed_forward).__name__ for l in model.layers] == ["SwiGLUFeedForward", "Top1Experts"] * 2
    assert model.layers[1].mixer.position_encoding.rotation().rotary_dim == 8
    assert model.layers[0].mixer.position_encoding.rotation().rotary_dim == 16
    assert model.layers[0].mixer.position_encoding.score_scale() == 1.0
    runner = ModelRunner(model, page_size=8, num_pages=16, max_num_seqs=2, poison=True)
    a, b = ru.random_ids(29, 77, 8), ru.random_ids(13, 77, 9)
    ref_a, ref_b = plain_routed(weights, cfg_dict, a), plain_routed(weights, cfg_dict, b)
    runner.admit("a")
    runner.admit("b")
    got_a, got_b = [], []
    got_a.append(runner.step([SeqEntry("a", a[:11], 0, list(range(11)))]))
    l = runner.step([SeqEntry("a", a[11:12], 11, [0]), SeqEntry("b", b[:7], 0, list(range(7)))])
    got_a.append(l[:1]); got_b.append(l[1:])
    l = runner.step([SeqEntry("b", b[7:8], 7, [0]), SeqEntry("a", a[12:], 12, list(range(17)))])
    got_b.append(l[:1]); got_a.append(l[1:])
    got_b.append(runner.step([SeqEntry("b", b[8:], 8, list(range(5)))]))
    scale = max(1.0, ref_a.abs().max().item())
    assert (torch.cat(got_a).cpu() - ref_a).abs().max().item() < 2e-4 * scale
    assert (torch.cat(got_b).cpu() - ref_b).abs().max().item() < 2e-4 * scale


# ----------------------------------------- a mixer that caches one tensor of a width of its own

def register_latent_toy():
    """A toy mixer that keeps ONE tensor per token in the paged cache (a latent of a width that is
    neither a head size nor a multiple of 16) and attends over it: it is key and value at once.
    Registered from here; the package's cache planning, page pools, block tables and step function
    serve it as they are."""
    from dispec_b200 import register_architecture, register_part
    from dispec_b200.config.model_config import ModelConfig
    from dispec_b200.models.spec import ModelSpec
    from dispec_b200.parts.base import CacheNeed, CacheTensor, Mixer, PartSpec, TensorSpec
    from dispec_b200.registry import architectures

    if "ToyLatentForCausalLM" in architectures():
        return

    @register_part("mixer", "toy_latent_attention")
    class LatentAttention(Mixer):
        """c_t = h_t Wc^T (cached); s_tj = (h_t Wq^T) . c_j / sqrt(latent) for j <= t;
        y_t = (sum_j softmax(s_t)_j c_j) Wo^T."""
        graph_safe = False  # walks the sequences of the step on the host

        def __init__(self, hidden_size, latent_size):
            self.h, self.l = hidden_size, latent_size

        def tensor_specs(self):
            return {"q.weight": TensorSpec((self.l, self.h)), "c.weight": TensorSpec((self.l, self.h)),
                    "o.weight": TensorSpec((self.h, self.l))}

        def load(self, tensors):
            self.wq, self.wc, self.wo = tensors["q.weight"], tensors["c.weight"], tensors["o.weight"]

        def cache_need(self):
            return CacheNeed((CacheTensor("latent", 1, self.l),), window=0)

        def forward(self, ctx, x, cache, state):
            assert set(cache.tensors) == {"latent"}
            pool = cache.tensors["latent"]  # [pages, 1, page_size, latent]
            assert pool.shape[1:] == (1, cache.page_size, self.l)
            q = x.float() @ self.wq.float().T
            c = (x.float() @ self.wc.float().T).to(pool.dtype)
            pos, seq = ctx.positions.long(), ctx.seq_of_token.long()
            page = cache.page_table[seq, pos // cache.page_size].long()
            pool[page, 0, pos % cache.page_size] = c
            out = torch.empty_like(q)
            for s in range(ctx.num_seqs):
                a, b, n = ctx.host_q_start[s], ctx.host_q_start[s + 1], ctx.host_ctx_len[s]
                pages = cache.page_table[s, :(n + cache.page_size - 1) // cache.page_size].long()
                keys = pool[pages, 0].reshape(-1, self.l)[:n].float()  # every stored latent of the request
                scores = q[a:b] @ keys.T / self.l ** 0.5
                first = n - (b - a)  # position of the portion's first token
                hidden = torch.arange(n, device=x.device)[None, :] > (first + torch.arange(b - a, device=x.device))[:, None]
                out[a:b] = torch.softmax(scores.masked_fill(hidden, float("-inf")), dim=-1) @ keys
            return (out @ self.wo.float().T).to(x.dtype)

    @dataclass(frozen=True)
    class LatentConfig(ModelConfig):
        architecture: ClassVar[str] = "ToyLatentForCausalLM"
        vocab_size: int = 0
        hidden_size: int = 0
        latent_size: int = 0
        intermediate_size: int = 0
        num_layers: int = 0
        eps: float = 0.0
        KEYS: ClassVar[tuple] = ("vocab_size", "hidden_size", "latent_size", "intermediate_size", "num_layers", "eps")

        @classmethod
        def from_dict(cls, d):
            return cls(**{k: d[k] for k in cls.KEYS})

        def to_dict(self):
            return dict(architectures=[self.architecture], **{k: getattr(self, k) for k in self.KEYS})

    def build(cfg):
        h = cfg.hidden_size
        layers = []
        for i in range(cfg.num_layers):
            p = f"layers.{i}."
            norm = lambda n: PartSpec("norm", "rms_norm", {"hidden_size": h, "eps": cfg.eps}, {"weight": p + n})
            mixer = PartSpec("mixer", "toy_latent_attention", {"hidden_size": h, "latent_size": cfg.latent_size},
                             {f"{n}.weight": f"{p}mix.{n}" for n in "qco"})
            ffn = PartSpec("feed_forward", "swiglu", {"hidden_size": h, "intermediate_size": cfg.intermediate_size},
                           {f"{n}_proj.weight": p + "ffn." + n for n in ("gate", "up", "down")})
            layers.append(PartSpec("block", "pre_norm", {"mixer_norm": norm("n1"), "mixer": mixer,
                                                         "ffn_norm": norm("n2"), "feed_forward": ffn}))
        return ModelSpec("ToyLatentForCausalLM",
                         PartSpec("embedding", "token_embedding", {"vocab_size": cfg.vocab_size, "hidden_size": h}, {"weight": "emb"}),
                         layers,
                         PartSpec("norm", "rms_norm", {"hidden_size": h, "eps": cfg.eps}, {"weight": "final"}),
                         PartSpec("head", "linear_head", {"vocab_size": cfg.vocab_size, "hidden_size": h}, {"weight": "emb"}),
                         vocab_size=cfg.vocab_size, max_position=4096)

    register_architecture("ToyLatentForCausalLM", LatentConfig, build)


def plain_latent(weights, cfg, ids, cache_dtype):
    T, l = len(ids), cfg["latent_size"]
    x = weights["emb"][torch.as_tensor(ids)]
    visible = torch.arange(T)[None, :] <= torch.arange(T)[:, None]
    for i in range(cfg["num_layers"]):
        p = f"layers.{i}."
        h = plain.rms_norm(x, weights[p + "n1"], cfg["eps"])
        q = h @ weights[p + "mix.q"].T
        c = (h @ weights[p + "mix.c"].T).to(cache_dtype).float()
        s = (q @ c.T / l ** 0.5).masked_fill(~visible, float("-inf"))
        x = x + (torch.softmax(s, dim=-1) @ c) @ weights[p + "mix.o"].T
        h = plain.rms_norm(x, weights[p + "n2"], cfg["eps"])
        x = x + plain.swiglu_mlp(h, weights[p + "ffn.gate"], weights[p + "ffn.up"], weights[p + "ffn.down"])
    return plain.rms_norm(x, weights["final"], cfg["eps"]) @ weights["emb"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_mixer_that_caches_one_latent_tensor(tmp_path, dtype):
    """The cache a mixer asks for is a list of named tensors, each with its own heads and width:
    one latent of width 24 here instead of a key and a value.  Two requests, cut anywhere, with
    so few pages that a finished request's pages are used again (freed pages hold NaN)."""
    from safetensors.torch import load_file
    from dispec_b200 import load_model, load_model_config, write_random_model
    from dispec_b200.engine import ModelRunner, SeqEntry
    register_latent_toy()
    cfg_dict = dict(architectures=["ToyLatentForCausalLM"], vocab_size=83, hidden_size=40, latent_size=24,
                    intermediate_size=64, num_layers=2, eps=1e-5)
    cfg = load_model_config(cfg_dict)
    write_random_model(cfg, str(tmp_path), seed=11, std=0.2, dtype="bfloat16")
    weights = {k: v.float() for k, v in load_file(str(tmp_path / "model.safetensors")).items()}
    model = load_model(str(tmp_path), dtype, DEV)
    group = model.cache_groups[0]
    assert len(model.cache_groups) == 1 and group.num_slots == 2
    assert [(t.name, t.num_heads, t.width) for t in group.tensors] == [("latent", 1, 24)]
    assert group.page_elements(8) == 2 * 8 * 24
    runner = ModelRunner(model, page_size=8, num_pages=6, max_num_seqs=2, poison=True)
    assert set(runner.storage.pools[0]) == {"latent"} and runner.storage.pools[0]["latent"].shape == (2, 6, 1, 8, 24)
    cache_dtype = torch.float32 if dtype == "float32" else torch.bfloat16
    a, b, c = ru.random_ids(27, 83, 1), ru.random_ids(13, 83, 2), ru.random_ids(19, 83, 3)
    ref = {n: plain_latent(weights, cfg_dict, ids, cache_dtype) for n, ids in (("a", a), ("b", b), ("c", c))}
    got = {"a": [], "b": [], "c": []}
    runner.admit("a")
    runner.admit("b")
    got["a"].append(runner.step([SeqEntry("a", a[:10], 0, list(range(10)))]))
    l = runner.step([SeqEntry("a", a[10:11], 10, [0]), SeqEntry("b", b[:9], 0, list(range(9)))])
    got["a"].append(l[:1]); got["b"].append(l[1:])
    l = runner.step([SeqEntry("b", b[9:10], 9, [0]), SeqEntry("a", a[11:], 11, list(range(16)))])
    got["b"].append(l[:1]); got["a"].append(l[1:])
    got["b"].append(runner.step([SeqEntry("b", b[10:], 10, list(range(3)))]))
    runner.release("a")  # four pages go back, filled with NaN, and are handed to c
    runner.admit("c")
    got["c"].append(runner.step([SeqEntry("c", c[:17], 0, list(range(17)))]))
    got["c"].append(runner.step([SeqEntry("c", c[17:], 17, [0, 1])]))
    tol = 2e-4 if dtype == "float32" else 0.06
    for name in got:
        out = torch.cat(got[name]).cpu()
        assert torch.isfinite(out).all()
        scale = max(1.0, ref[name].abs().max().item())
        assert (out - ref[name]).abs().max().item() < tol * scale, name
    runner.release("b")
    runner.release("c")
    runner.cache.check()
    assert runner.cache.num_free_pages(0) == 6
