"""More parts the framework has never seen, defined and registered here: a
feed-forward with routing (top-1 of a few experts), another position encoding
(a learned offset added to queries and keys, which also has to write the
cache itself), and another block arrangement (mixer and feed-forward in
parallel off one norm).  An architecture registered here uses them layer by
layer beside the package's own parts.  Nothing in the package's files changes.
Checked against a plain whole-sequence implementation of the same toy model."""
import pytest
import torch

import fixtures
import plain_llama
from lyapunov_engine_b200 import LLMEngine, SamplingParams, load_model, register_architecture
from lyapunov_engine_b200.parts import (FEED_FORWARDS, MIXERS, NORMS, Block, FeedForward, LayerSpec, ModelSpec, PartSpec,
                                        PositionEncoding, RunSpec, TensorDecl, register_block, register_feed_forward,
                                        register_position_encoding)

pytestmark = pytest.mark.gpu

H, V, I, NH, NKV, HD, WINDOW, EXPERTS, MAXPOS = 40, 97, 56, 4, 2, 16, 5, 3, 128


@register_feed_forward("toy_routed")
class ToyRoutedFeedForward(FeedForward):
    """Router logits in 32 bits, softmax, the best expert alone (weighted by
    its probability): y = p_e * W2_e relu(W1_e x)."""

    def __init__(self, hidden_size, inner_size, experts, prefix):
        self.hidden_size, self.inner_size, self.experts, self.prefix = hidden_size, inner_size, experts, prefix

    def tensors(self):
        decls = [TensorDecl(self.prefix + "router", (self.experts, self.hidden_size))]
        for e in range(self.experts):
            decls += [TensorDecl(f"{self.prefix}w1.{e}", (self.inner_size, self.hidden_size)),
                      TensorDecl(f"{self.prefix}w2.{e}", (self.hidden_size, self.inner_size))]
        return decls

    def bind(self, get, runtime):
        self.router = get(self.prefix + "router")
        self.w1 = [get(f"{self.prefix}w1.{e}") for e in range(self.experts)]
        self.w2 = [get(f"{self.prefix}w2.{e}") for e in range(self.experts)]

    def forward(self, x, ctx):
        probs = torch.softmax(x.float() @ self.router.float().t(), dim=-1)
        best = probs.argmax(dim=-1)
        y = torch.zeros_like(x, dtype=torch.float32)
        for e in range(self.experts):
            rows = (best == e).nonzero().flatten()
            if rows.numel():
                hidden = torch.relu(x[rows].float() @ self.w1[e].float().t())
                y[rows] = probs[rows, e:e + 1] * (hidden @ self.w2[e].float().t())
        return y.to(x.dtype)


@register_position_encoding("toy_offset")
class ToyOffsetEncoding(PositionEncoding):
    """q_h += P[pos], k_h += P[pos] for every head; then keys and values go to
    their place in the paged cache through the block table."""

    def __init__(self, head_dim, max_positions, table_name):
        self.head_dim, self.max_positions, self.table_name = head_dim, max_positions, table_name

    def tensors(self):
        return [TensorDecl(self.table_name, (self.max_positions, self.head_dim))]

    def bind(self, get, runtime):
        self.table = get(self.table_name)

    def encode_and_store(self, qkv, geometry, ctx, kv, write):
        nh, nkv, hd = geometry
        T = qkv.shape[0]
        pos = ctx.positions.long()
        heads = qkv.view(T, nh + 2 * nkv, hd)
        heads[:, :nh + nkv] += self.table[pos].to(qkv.dtype).unsqueeze(1)
        if write and kv is not None:
            table = ctx.block_tables[kv.group].long()
            page = table[ctx.request_of_token.long(), pos // kv.page_size]
            kv.k[page, :, pos % kv.page_size] = heads[:, nh:nh + nkv]
            kv.v[page, :, pos % kv.page_size] = heads[:, nh + nkv:]


@register_block("toy_parallel")
class ToyParallelBlock(Block):
    """h = h + mixer(norm(h)) + feed_forward(norm(h)): one norm, both branches read it."""

    def __init__(self, mixer, feed_forward, norm):
        self.mixer = MIXERS.build(mixer)
        self.feed_forward = FEED_FORWARDS.build(feed_forward)
        self.norm = NORMS.build(norm)

    def tensors(self):
        return self.norm.tensors() + self.mixer.tensors() + self.feed_forward.tensors()

    def bind(self, get, runtime):
        for p in (self.norm, self.mixer, self.feed_forward):
            p.bind(get, runtime)

    def forward(self, stream, ctx, cache):
        n = self.norm.apply(stream.resid, stream.pending, workspace=ctx.workspace)
        a = self.mixer.forward(n, ctx, cache)
        if a.dim() == 3:                  # partial sums of a split product
            a = a.sum(0)
        stream.pending = (a.float() + self.feed_forward.forward(n, ctx).float()).to(n.dtype)


def toy_spec(raw):
    def attention(p, window, position):
        return PartSpec("attention", {
            "hidden_size": H, "num_heads": NH, "num_kv_heads": NKV, "head_dim": HD, "window": window, "position": position,
            "q_name": p + "q", "k_name": p + "k", "v_name": p + "v", "o_name": p + "o"})
    rotary = PartSpec("rotary", {"head_dim": HD, "theta": 10000.0, "max_positions": MAXPOS})
    offset = PartSpec("toy_offset", {"head_dim": HD, "max_positions": MAXPOS, "table_name": "layers.0.offsets"})

    def norm(name):
        return PartSpec("rmsnorm", {"hidden_size": H, "eps": 1e-5, "weight_name": name})

    def routed(p):
        return PartSpec("toy_routed", {"hidden_size": H, "inner_size": I, "experts": EXPERTS, "prefix": p + "ff."})
    gated = PartSpec("gated_silu", {"hidden_size": H, "intermediate_size": I, "gate_name": "layers.0.gate",
                                    "up_name": "layers.0.up", "down_name": "layers.0.down"})
    layers = (
        LayerSpec(PartSpec("prenorm", {"mixer": attention("layers.0.", None, offset), "feed_forward": gated,
                                       "mixer_norm": norm("layers.0.norm1"), "feed_forward_norm": norm("layers.0.norm2")})),
        LayerSpec(PartSpec("toy_parallel", {"mixer": attention("layers.1.", None, rotary), "feed_forward": routed("layers.1."),
                                            "norm": norm("layers.1.norm")})),
        LayerSpec(PartSpec("prenorm", {"mixer": attention("layers.2.", WINDOW, rotary), "feed_forward": routed("layers.2."),
                                       "mixer_norm": norm("layers.2.norm1"), "feed_forward_norm": norm("layers.2.norm2")})),
    )
    return ModelSpec(architecture="ToyRoutedForCausalLM", hidden_size=H, vocab_size=V, max_positions=MAXPOS,
                     embedding=PartSpec("token_embedding", {"vocab_size": V, "hidden_size": H, "weight_name": "embed"}),
                     layers=layers, run_order=(RunSpec(0), RunSpec(1), RunSpec(2)), final_norm=norm("norm"),
                     head=PartSpec("linear_head", {"vocab_size": V, "hidden_size": H, "weight_name": "head", "tied_to": None}),
                     config_json=dict(raw))


register_architecture("ToyRoutedForCausalLM", toy_spec)
TOY_CONFIG = {"architectures": ["ToyRoutedForCausalLM"]}


def plain_toy(w, ids):
    """Whole sequence, no cache, float32."""
    T = len(ids)
    h = w["embed"][torch.tensor(ids)]
    inv = plain_llama.plain_inv_freq(HD, 10000.0, None)
    cos, sin = plain_llama.plain_cos_sin(torch.arange(T), inv)

    def attn(x, p, window, offsets=None):
        q = (x @ w[p + "q"].T).view(T, NH, HD).transpose(0, 1)
        k = (x @ w[p + "k"].T).view(T, NKV, HD).transpose(0, 1)
        v = (x @ w[p + "v"].T).view(T, NKV, HD).transpose(0, 1)
        if offsets is None:
            q, k = plain_llama.plain_rotate_half(q, cos, sin), plain_llama.plain_rotate_half(k, cos, sin)
        else:
            q, k = q + offsets[:T], k + offsets[:T]
        o = plain_llama.plain_attention(q, k, v, window).transpose(0, 1).reshape(T, NH * HD)
        return o @ w[p + "o"].T

    def routed(x, p):
        probs = torch.softmax(x @ w[p + "ff.router"].T, dim=-1)
        best = probs.argmax(-1)
        rows = []
        for t in range(T):
            e = int(best[t])
            rows.append(probs[t, e] * (torch.relu(x[t] @ w[f"{p}ff.w1.{e}"].T) @ w[f"{p}ff.w2.{e}"].T))
        return torch.stack(rows)

    def rms(x, name):
        return plain_llama.plain_rmsnorm(x, w[name], 1e-5)

    h = h + attn(rms(h, "layers.0.norm1"), "layers.0.", None, w["layers.0.offsets"])
    h = h + plain_llama.plain_mlp(rms(h, "layers.0.norm2"), w["layers.0.gate"], w["layers.0.up"], w["layers.0.down"])
    n = rms(h, "layers.1.norm")
    h = h + attn(n, "layers.1.", None) + routed(n, "layers.1.")
    h = h + attn(rms(h, "layers.2.norm1"), "layers.2.", WINDOW)
    h = h + routed(rms(h, "layers.2.norm2"), "layers.2.")
    return rms(h, "norm") @ w["head"].T


@pytest.fixture(scope="module")
def toy(tmp_path_factory):
    from lyapunov_engine_b200.weights import write_random_model
    folder = str(tmp_path_factory.mktemp("toy_routed"))
    write_random_model(folder, TOY_CONFIG, seed=9, dtype=torch.float32, std=0.15, norm_jitter=0.1)
    _, w = plain_llama.read_model_folder(folder)
    assert "layers.1.ff.w2.2" in w and w["layers.0.offsets"].shape == (MAXPOS, HD)
    return folder, w


def test_routed_offset_parallel_model_steps_through_the_framework(toy):
    from lyapunov_engine_b200 import build
    from lyapunov_engine_b200.cache import DeviceCache
    from lyapunov_engine_b200.engine.step import ModelRunner
    folder, w = toy
    host = build.load_host()
    loaded = load_model(folder, "float32", "cuda:0", max_model_len=MAXPOS)
    assert [(g.window, g.num_kv_heads) for g in loaded.model.groups] == [(None, NKV), (WINDOW, NKV)]
    cache = DeviceCache(loaded.model, loaded.runtime, num_blocks=40, block_size=4, max_num_seqs=2)
    runner = ModelRunner(loaded.model, cache, loaded.runtime, 96, 2, MAXPOS, use_cuda_graphs=False, check_status=True)
    requests = {0: fixtures.random_ids({"vocab_size": V}, 41, 11), 1: fixtures.random_ids({"vocab_size": V}, 58, 12)}
    ref = {r: plain_toy(w, ids) for r, ids in requests.items()}
    # every expert is used somewhere, or the routing is not tested
    probe = plain_llama.plain_rmsnorm(w["embed"][torch.tensor(requests[1])], w["layers.1.norm"], 1e-5) @ w["layers.1.ff.router"].T
    assert probe.argmax(-1).unique().numel() >= 2
    seqs = {r: host.Sequence(r, ids, host.SamplingParams()) for r, ids in requests.items()}
    got = {r: [] for r in requests}
    sizes = {0: [9, 1, 1, 14, 2, 14], 1: [2, 30, 1, 1, 1, 23]}
    for step in range(6):
        entries = []
        for r in requests:
            n, start = sizes[r][step], seqs[r].get_num_computed_tokens()
            assert cache.manager.grow(seqs[r], start + n)
            entries.append(host.StepEntry(seqs[r], start, n, list(range(n))))
        logits = runner.step(entries).cpu()
        row = 0
        for e in entries:
            got[e.seq.get_seq_id()].append(logits[row:row + e.count])
            row += e.count
            e.seq.set_num_computed_tokens(e.start + e.count)
            cache.manager.release_passed(e.seq)
        assert cache.manager.audit() == ""
    for r in requests:
        torch.testing.assert_close(torch.cat(got[r]), ref[r], atol=2e-4, rtol=2e-4)


def test_routed_offset_parallel_model_generates(toy):
    folder, w = toy
    engine = LLMEngine.from_pretrained(folder, dtype="float32", num_blocks=24, block_size=4, max_num_seqs=2,
                                       max_num_batched_tokens=16, use_cuda_graphs=False, max_model_len=MAXPOS)
    prompts = [fixtures.random_ids({"vocab_size": V}, n, 70 + n) for n in (5, 22)]
    outs = engine.generate(prompts, SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))
    for p, o in zip(prompts, outs):
        ids, want = list(p), []
        for _ in range(6):
            t = int(plain_toy(w, ids)[-1].argmax())
            want.append(t)
            ids.append(t)
        assert o.output_tokens == want
    assert engine.block_manager.audit() == ""
