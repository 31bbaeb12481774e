"""The framework takes parts it has never seen: a toy mixer with state of its
own (defined here), an architecture (registered here) that mixes it with
windowed and full attention layer by layer, runs one layer twice and lets one
run read the pages another run wrote.  Nothing in the package's files changes.
Checked against a plain whole-sequence implementation of the same toy model."""
import pytest
import torch

import fixtures
import plain_llama
from lyapunov_engine_b200 import EngineConfig, LLMEngine, SamplingParams, load_model, register_architecture
from lyapunov_engine_b200.parts import (LayerSpec, Mixer, ModelSpec, PartSpec, RunSpec, StateNeed, TensorDecl,
                                        register_mixer)

pytestmark = pytest.mark.gpu

H, V, I, NH, NKV, HD, WINDOW = 48, 131, 80, 4, 2, 16, 6
DECAY = 0.8


@register_mixer("toy_decay")
class ToyDecayMixer(Mixer):
    """s_t = decay * s_{t-1} + x_t W_in^T;  y_t = s_t W_out^T.  The state s of
    each request lives in its state slot between steps.  It never clears a
    slot itself: the framework hands a request's first step a zeroed row,
    whoever held the slot before."""

    def __init__(self, hidden_size, decay, in_name, out_name):
        self.hidden_size, self.decay, self.names = hidden_size, decay, (in_name, out_name)

    def state_need(self):
        return StateNeed((self.hidden_size,), torch.float32)

    def tile_sizes(self):
        return [8]       # a tile size no kernel of the package uses: the step's integers list it because this mixer asks

    def tensors(self):
        return [TensorDecl(n, (self.hidden_size, self.hidden_size)) for n in self.names]

    def bind(self, get, runtime):
        self.w_in, self.w_out = (get(n) for n in self.names)
        self.runtime = runtime

    def forward(self, x, ctx, cache):
        cu, slots = ctx.cu_q.tolist(), ctx.state_slots.tolist()
        tile_request, tile_q0, num_tiles, _ = ctx.tiles[8]
        assert num_tiles == sum((cu[b + 1] - cu[b] + 7) // 8 for b in range(ctx.num_requests))
        assert sorted(zip(tile_request.tolist(), tile_q0.tolist())) == \
            sorted((b, q0) for b in range(ctx.num_requests) for q0 in range(0, cu[b + 1] - cu[b], 8))
        u = (x.float() @ self.w_in.float().t())
        y = torch.empty_like(u)
        for b in range(ctx.num_requests):
            if slots[b] < 0:
                continue
            s = cache.state[slots[b]]
            for t in range(cu[b], cu[b + 1]):
                s = self.decay * s + u[t]
                y[t] = s
            cache.state[slots[b]] = s
        return (y @ self.w_out.float().t()).to(x.dtype)


def toy_spec(raw):
    def attention(p, window):
        return PartSpec("attention", {
            "hidden_size": H, "num_heads": NH, "num_kv_heads": NKV, "head_dim": HD, "window": window,
            "position": PartSpec("rotary", {"head_dim": HD, "theta": 10000.0, "max_positions": 256}),
            "q_name": p + "q", "k_name": p + "k", "v_name": p + "v", "o_name": p + "o"})

    def block(i, mixer):
        p = f"layers.{i}."
        ff = PartSpec("gated_silu", {"hidden_size": H, "intermediate_size": I, "gate_name": p + "gate",
                                     "up_name": p + "up", "down_name": p + "down"})
        n1 = PartSpec("rmsnorm", {"hidden_size": H, "eps": 1e-5, "weight_name": p + "norm1"})
        n2 = PartSpec("rmsnorm", {"hidden_size": H, "eps": 1e-5, "weight_name": p + "norm2"})
        return LayerSpec(PartSpec("prenorm", {"mixer": mixer, "feed_forward": ff, "mixer_norm": n1,
                                              "feed_forward_norm": n2}))
    layers = (block(0, attention("layers.0.", None)),
              block(1, PartSpec("toy_decay", {"hidden_size": H, "decay": DECAY, "in_name": "layers.1.in",
                                              "out_name": "layers.1.out"})),
              block(2, attention("layers.2.", WINDOW)),
              block(3, attention("layers.3.", None)))
    # layer 0 runs twice (each run has pages of its own); the last run reads the pages of the first
    order = (RunSpec(0), RunSpec(1), RunSpec(2), RunSpec(0), RunSpec(3, reads_cache_of=0))
    return ModelSpec(architecture="ToyForCausalLM", hidden_size=H, vocab_size=V, max_positions=256,
                     embedding=PartSpec("token_embedding", {"vocab_size": V, "hidden_size": H, "weight_name": "embed"}),
                     layers=layers, run_order=order,
                     final_norm=PartSpec("rmsnorm", {"hidden_size": H, "eps": 1e-5, "weight_name": "norm"}),
                     head=PartSpec("linear_head", {"vocab_size": V, "hidden_size": H, "weight_name": "head",
                                                   "tied_to": "embed"}),
                     config_json=dict(raw))


register_architecture("ToyForCausalLM", toy_spec)
TOY_CONFIG = {"architectures": ["ToyForCausalLM"]}


def plain_toy(w, ids):
    """Whole sequence, no cache, float32."""
    T = len(ids)
    h = w["embed"][torch.tensor(ids)]
    inv = plain_llama.plain_inv_freq(HD, 10000.0, None)
    cos, sin = plain_llama.plain_cos_sin(torch.arange(T), inv)
    kept = {}

    def attn(x, p, window, read=None, keep=None):
        q = (x @ w[p + "q"].T).view(T, NH, HD).transpose(0, 1)
        q = plain_llama.plain_rotate_half(q, cos, sin)
        if read is None:
            k = plain_llama.plain_rotate_half((x @ w[p + "k"].T).view(T, NKV, HD).transpose(0, 1), cos, sin)
            v = (x @ w[p + "v"].T).view(T, NKV, HD).transpose(0, 1)
            if keep is not None:
                kept[keep] = (k, v)
        else:
            k, v = kept[read]
        o = plain_llama.plain_attention(q, k, v, window).transpose(0, 1).reshape(T, NH * HD)
        return o @ w[p + "o"].T

    def decay(x):
        u = x @ w["layers.1.in"].T
        s = torch.zeros(H)
        out = []
        for t in range(T):
            s = DECAY * s + u[t]
            out.append(s)
        return torch.stack(out) @ w["layers.1.out"].T

    def block(h, i, mixer):
        p = f"layers.{i}."
        h = h + mixer(plain_llama.plain_rmsnorm(h, w[p + "norm1"], 1e-5))
        n = plain_llama.plain_rmsnorm(h, w[p + "norm2"], 1e-5)
        return h + plain_llama.plain_mlp(n, w[p + "gate"], w[p + "up"], w[p + "down"])

    h = block(h, 0, lambda x: attn(x, "layers.0.", None, keep="first"))
    h = block(h, 1, decay)
    h = block(h, 2, lambda x: attn(x, "layers.2.", WINDOW))
    h = block(h, 0, lambda x: attn(x, "layers.0.", None))
    h = block(h, 3, lambda x: attn(x, "layers.3.", None, read="first"))
    return plain_llama.plain_rmsnorm(h, w["norm"], 1e-5) @ w["embed"].T


@pytest.fixture(scope="module")
def toy(tmp_path_factory):
    from lyapunov_engine_b200.models.model import Model
    from lyapunov_engine_b200.weights import write_random_model
    folder = str(tmp_path_factory.mktemp("toy"))
    write_random_model(folder, TOY_CONFIG, seed=5, dtype=torch.float32, std=0.12, norm_jitter=0.1)
    model = Model(toy_spec(TOY_CONFIG))
    # what the cache must hold follows from the description alone
    assert [(g.window, g.num_kv_heads) for g in model.groups] == [(None, NKV), (WINDOW, NKV)]
    assert model.streams_per_group == [2, 1] and len(model.states) == 1
    assert model.tile_sizes == [8, 16, 128]     # the toy mixer's and the attention kernels'
    assert [(r.group, r.stream, r.writes, r.state) for r in model.runs] == \
        [(0, 0, True, None), (None, None, True, 0), (1, 0, True, None), (0, 1, True, None), (0, 0, False, None)]
    _, w = plain_llama.read_model_folder(folder)
    return folder, w


def test_toy_model_steps_through_the_framework(toy):
    from lyapunov_engine_b200 import build
    from lyapunov_engine_b200.cache import DeviceCache
    from lyapunov_engine_b200.engine.step import ModelRunner
    folder, w = toy
    host = build.load_host()
    loaded = load_model(folder, "float32", "cuda:0", max_model_len=128)
    cache = DeviceCache(loaded.model, loaded.runtime, num_blocks=40, block_size=4, max_num_seqs=3)
    runner = ModelRunner(loaded.model, cache, loaded.runtime, 128, 3, 96, use_cuda_graphs=False, check_status=True)
    requests = {0: fixtures.random_ids({"vocab_size": V}, 45, 1), 1: fixtures.random_ids({"vocab_size": V}, 30, 2),
                2: fixtures.random_ids({"vocab_size": V}, 61, 3)}
    ref = {r: plain_toy(w, ids) for r, ids in requests.items()}
    seqs = {r: host.Sequence(r, ids, host.SamplingParams()) for r, ids in requests.items()}
    got = {r: [] for r in requests}
    sizes = {0: [7, 2, 16, 1, 1, 3, 15], 1: [30], 2: [1, 1, 9, 2, 20, 1, 1, 26]}
    cursor = {r: 0 for r in requests}
    window_pages_peak = 0
    while any(cursor[r] < len(sizes[r]) for r in requests):
        entries = []
        for r in requests:
            if cursor[r] < len(sizes[r]):
                n, start = sizes[r][cursor[r]], seqs[r].get_num_computed_tokens()
                assert cache.manager.grow(seqs[r], start + n)
                entries.append(host.StepEntry(seqs[r], start, n, list(range(n))))
                cursor[r] += 1
        logits = runner.step(entries).cpu()
        row = 0
        for e in entries:
            got[e.seq.get_seq_id()].append(logits[row:row + e.count])
            row += e.count
            e.seq.set_num_computed_tokens(e.start + e.count)
            cache.manager.release_passed(e.seq)
        window_pages_peak = max(window_pages_peak, cache.manager.get_num_used_blocks(1))
        assert cache.manager.audit() == ""
    for r in requests:
        out = torch.cat(got[r])
        assert out.shape == ref[r].shape
        torch.testing.assert_close(out, ref[r], atol=2e-4, rtol=2e-4)
    # the window's group gave pages back while the requests lived
    assert window_pages_peak < cache.manager.get_num_used_blocks(0) // 2
    for s in seqs.values():
        cache.manager.free(s)
    assert cache.manager.get_num_free_blocks(0) == 40 and cache.manager.get_num_free_blocks(1) == 40


def test_toy_model_generates_through_the_entry_point(toy):
    folder, w = toy
    # two state slots for five requests: the later ones get slots that others have left their state in
    engine = LLMEngine.from_pretrained(folder, dtype="float32", num_blocks=24, block_size=4, max_num_seqs=2,
                                       max_num_batched_tokens=16, use_cuda_graphs=False, max_model_len=96)
    prompts = [fixtures.random_ids({"vocab_size": V}, n, 40 + n) for n in (3, 19, 26, 1, 11)]
    outs = engine.generate(prompts, SamplingParams(temperature=0.0, max_tokens=7, ignore_eos=True))
    for p, o in zip(prompts, outs):
        ids, want = list(p), []
        for _ in range(7):
            t = int(plain_toy(w, ids)[-1].argmax())
            want.append(t); ids.append(t)
        assert o.output_tokens == want and o.finish_reason == "length"
    assert engine.block_manager.audit() == ""
