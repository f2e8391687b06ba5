"""Parts alone against the plain implementation, and the generality of the layer machinery:
a toy mixer with state of its own registered from this file, a layer that runs twice, a run that
reads another run's cache, and a windowed mixer in one layer only - none of them a model of anyone's."""

import random

import pytest
import torch

import helpers as H
import plain_llama as pl

pytestmark = pytest.mark.gpu
F64 = torch.float64


def _runner(model, page_tokens, max_tokens, max_live=4, num_pages=None, **opts):
    from bare_cuda_4gib_b200.cache.manager import CacheManager
    from bare_cuda_4gib_b200.engine.step import StepRunner

    cap = -(-max_tokens // page_tokens) * page_tokens
    cache = CacheManager(model.cache_demands(), page_tokens=page_tokens, max_seqs=max_live, max_tokens=cap,
                         num_pages=num_pages or (max_live * cap // page_tokens), dtype=model.dtype, device="cuda")
    return StepRunner(model, cache, max_step_tokens=cap, max_batch_seqs=max_live, **opts), cache


def _llama(name, dtype, mutate=None):
    """The tiny configuration's model, optionally with its spec changed before the parts are built."""
    import bare_cuda_4gib_b200.models  # noqa: F401
    from bare_cuda_4gib_b200.config import LlamaConfig, resolve_architecture
    from bare_cuda_4gib_b200.engine.model import load_model_with_spec

    cfg = LlamaConfig.from_dict(H.TINY[name][0])
    spec = resolve_architecture(H.TINY[name][0]).build_spec(cfg)
    if mutate:
        mutate(spec)
    return load_model_with_spec(H.model_folder(name), spec, dtype, "cuda"), cfg


def _tol(dtype):
    return 1e-5 if dtype == "float32" else 3e-2


def _err(got, want):
    got, want = got.double().cpu(), want.double().cpu()
    return float((got - want).abs().max() / want.abs().max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_each_part_alone(name, dtype):
    """norm, mixer, feed-forward, block, embedding and head, each called by itself on given inputs."""
    from bare_cuda_4gib_b200.engine.step import StepEntry
    from bare_cuda_4gib_b200.kernels.lib import Partials

    model, cfg = _llama(name, dtype)
    plain = H.plain_model(H.model_folder(name))
    page = H.TINY[name][1]
    runner, cache = _runner(model, page, 64, use_cuda_graphs=False)
    rng = random.Random(2)
    lens = [23, 9]
    ids = [H.random_ids(rng, n, cfg.vocab_size) for n in lens]
    slots = [cache.acquire_slot() for _ in lens]
    entries = [StepEntry(s, t, [len(t) - 1]) for s, t in zip(slots, ids)]
    runner.begin(entries)
    ctx, n, hid = runner.ctx, sum(lens), cfg.hidden_size
    act = model.dtype
    layer, pl_layer = model.blocks[1], plain.layers[1]
    positions = torch.cat([torch.arange(k) for k in lens])

    # embedding
    x = model.embed.forward(ctx)
    want_x = pl.embedding(plain.embed, torch.tensor(ids[0] + ids[1]))
    assert torch.equal(x[:n].cpu().double(), want_x)

    # norm with a pending contribution in two partial results
    res = torch.randn(n, hid, device="cuda")
    delta = torch.randn(2, n, hid, device="cuda")
    res_in = res.clone()
    h = layer.mixer_norm.forward(ctx, res, Partials(delta, 2), n)
    want_res = res_in.double().cpu() + delta.double().sum(0).cpu()
    assert _err(res, want_res) < 1e-6
    assert _err(h, pl.rms_norm(want_res, pl_layer.input_norm, plain.rms_norm_eps)) < (1e-5 if dtype == "float32" else 8e-3)

    # mixer (attention over the cache it has just written), one request after the other in the plain version
    hin = (0.5 * torch.randn(n, hid, device="cuda")).to(act)
    mixed = layer.mixer.forward(ctx, ctx.calls[1], hin)
    got = mixed.tensor.float().sum(0) if mixed.n > 1 else mixed.tensor.float()
    want, at = [], 0
    for k in lens:
        out, _ = pl.attention_mixer(plain, pl_layer, hin[at: at + k].double().cpu(), torch.arange(k))
        want.append(out)
        at += k
    assert _err(got[:n], torch.cat(want)) < _tol(dtype)

    # feed-forward
    ff = layer.ffn.forward(ctx, hin)
    got = ff.tensor.float().sum(0) if ff.n > 1 else ff.tensor.float()
    assert _err(got[:n], pl.feed_forward(pl_layer, hin.double().cpu())) < _tol(dtype)

    # block: residual in, residual + both contributions out (the last one still pending)
    res = (0.5 * torch.randn(n, hid, device="cuda"))
    res_in = res.clone()
    pending = layer.forward(ctx, ctx.calls[1], res, None)
    got = res.double() + (pending.tensor.double().sum(0) if pending.n > 1 else pending.tensor.double())
    want, at = [], 0
    for k in lens:
        out, _ = pl.decoder_block(plain, pl_layer, res_in[at: at + k].double().cpu(), torch.arange(k))
        want.append(out)
        at += k
    assert _err(got[:n], torch.cat(want)) < _tol(dtype)

    # final norm on the wanted rows + head
    res = torch.randn(n, hid, device="cuda")
    normed = model.final_norm.forward(ctx, res, None, ctx.n_want, ctx.want_rows, buffer="final_normed")
    logits = model.head.forward(ctx, normed, ctx.n_want)
    rows = [lens[0] - 1, n - 1]
    want = pl.output_head(plain, res[rows].double().cpu())
    assert _err(logits[:2], want) < _tol(dtype)


# ------------------------------------------------------------------------------ run order as data


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layer_named_twice_and_borrowed_cache(dtype):
    from bare_cuda_4gib_b200.parts.spec import LayerCall

    order = [(0, None), (1, None), (0, None), (1, 1)]

    def mutate(spec):
        spec.order = [LayerCall(l, c) for l, c in order]

    model, cfg = _llama("A", dtype, mutate)
    assert len(model.cache_demands()) == 4
    runner, cache = _runner(model, 16, 96)
    assert len(cache.groups) == 1 and cache.groups[0].members == [(0, 0), (1, 0), (2, 0)]     # the fourth run owns no cache
    plain = pl.read_model_folder(H.model_folder("A"))
    plain.order = order
    rng = random.Random(4)
    ids = H.random_ids(rng, 70, cfg.vocab_size)
    want = pl.forward_logits(plain, ids)
    from bare_cuda_4gib_b200.engine.step import StepEntry
    slot = cache.acquire_slot()
    got, fed = [], 0
    for size in (19, 2, 30, 1, 1, 17):
        got.append(runner.step([StepEntry(slot, ids[fed: fed + size], list(range(size)))]).float().cpu().clone())
        fed += size
    got = torch.cat(got)
    for p in range(70):
        assert H.row_error(got[p], want[p]) < H.TOLERANCE[dtype], p


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_window_in_one_layer_gives_pages_back(dtype):
    window = 24

    def mutate(spec):
        spec.layers[1].mixer.params["window"] = window          # layer 1 only: two cache groups

    model, cfg = _llama("B", dtype, mutate)
    runner, cache = _runner(model, 16, 240, max_live=2, num_pages=30)
    assert len(cache.groups) == 2
    plain = pl.read_model_folder(H.model_folder("B"))
    plain.layers[1].window = window
    rng = random.Random(6)
    ids = H.random_ids(rng, 200, cfg.vocab_size)
    want = pl.forward_logits(plain, ids)
    from bare_cuda_4gib_b200.engine.step import StepEntry
    slot = cache.acquire_slot()
    got, fed, sizes = [], 0, [50, 3, 40, 1, 1, 1, 33, 2, 60, 9]
    held = []
    for size in sizes:
        got.append(runner.step([StepEntry(slot, ids[fed: fed + size], list(range(size)))]).float().cpu().clone())
        fed += size
        cache.check_consistency()
        held.append(cache.pages_in_use())
    got = torch.cat(got)
    for p in range(fed):
        assert H.row_error(got[p], want[p]) < H.TOLERANCE[dtype], p
    windowed = [g for g in cache.groups if g.request.window == window][0]
    full = [g for g in cache.groups if g.request.window is None][0]
    assert full.pool.pages_in_use == -(-200 // 16)
    assert windowed.pool.pages_in_use <= -(-(window + 9) // 16) + 1     # only the window's pages remain
    assert windowed.pool.acquired_total > windowed.pool.pages_in_use


# ------------------------------------------------------------------------------ a toy mixer with state


def test_toy_mixer_with_state_is_registered_built_and_stepped():
    """A mixer defined here - an exponential moving average of its inputs, kept per request in a
    state slot - is registered, put into one layer of a model beside attention layers, and stepped
    in portions and in a batch; the engine's files are not touched."""
    from bare_cuda_4gib_b200.config import LlamaConfig
    from bare_cuda_4gib_b200.engine.model import expected_weights
    from bare_cuda_4gib_b200.engine.step import StepEntry
    from bare_cuda_4gib_b200.kernels.lib import Partials
    from bare_cuda_4gib_b200.models.llama import llama_spec
    from bare_cuda_4gib_b200.parts import Part, PartSpec, StateRequest, register_mixer
    from bare_cuda_4gib_b200.weights import random_tensors

    @register_mixer("toy_moving_average")
    class MovingAverage(Part):
        graph_safe = False        # its forward loops over requests on the host

        def local_weights(self):
            h = self.params["hidden"]
            return {"out": ((h, h), "matrix")}

        def cache_request(self):
            return None           # no pages

        def state_request(self):
            return StateRequest((self.params["hidden"],), torch.float32)

        def forward(self, ctx, call, h):
            decay = self.params["decay"]
            out = torch.zeros(ctx.n_tokens, self.params["hidden"], device=h.device)
            row = 0
            for slot, n in zip(ctx.host_slots, ctx.host_q_len):
                state = call.state[slot]
                for t in range(n):
                    state.mul_(decay).add_(h[row].float(), alpha=1.0 - decay)
                    out[row] = self.tensors["out"].float() @ state
                    row += 1
            return Partials(out)

    cfg = LlamaConfig.from_dict(H.TINY_A)
    spec = llama_spec(cfg)
    decay = 0.75
    spec.layers[0].mixer = PartSpec("toy_moving_average", {"hidden": cfg.hidden_size, "decay": decay},
                                    {"out": "model.layers.0.toy.out.weight"})
    expected, model = expected_weights(spec)
    assert "model.layers.0.toy.out.weight" in expected and "model.layers.0.self_attn.q_proj.weight" not in expected
    tensors = {k: v.to("cuda", torch.float32) for k, v in random_tensors(expected, seed=5).items()}
    model.bind(tensors, torch.float32, "cuda")
    assert not model.graph_safe
    demands = model.cache_demands()
    assert demands[0][0].kv is None and demands[0][0].state is not None and demands[1][0].kv is not None
    runner, cache = _runner(model, 16, 64)
    assert cache.state_of(0) is not None and len(cache.groups) == 1 and cache.groups[0].members == [(1, 0)]

    # the same model, plainly: layer 0 with the moving average, layer 1 as the plain Llama layer
    t64 = {k: v.double().cpu() for k, v in tensors.items()}
    plain = pl.PlainModel(cfg.vocab_size, cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads,
                          cfg.head_dim, cfg.intermediate_size, cfg.rope_theta, cfg.rms_norm_eps,
                          t64["model.embed_tokens.weight"], t64["model.norm.weight"], t64["lm_head.weight"])

    def layer_of(i):
        p = f"model.layers.{i}."
        g = lambda n: t64.get(p + n)
        return pl.PlainLayer(g("input_layernorm.weight"), g("self_attn.q_proj.weight"), g("self_attn.k_proj.weight"),
                             g("self_attn.v_proj.weight"), g("self_attn.o_proj.weight"),
                             g("post_attention_layernorm.weight"), g("mlp.gate_proj.weight"),
                             g("mlp.up_proj.weight"), g("mlp.down_proj.weight"))

    def plain_forward(ids):
        x = pl.embedding(plain.embed, torch.tensor(ids))
        l0, l1 = layer_of(0), layer_of(1)
        h = pl.rms_norm(x, l0.input_norm, plain.rms_norm_eps)
        state, mixed = torch.zeros(cfg.hidden_size, dtype=F64), []
        for t in range(len(ids)):
            state = decay * state + (1 - decay) * h[t].float().double()   # the toy keeps float32 state
            mixed.append(t64["model.layers.0.toy.out.weight"] @ state)
        x = x + torch.stack(mixed)
        x = x + pl.feed_forward(l0, pl.rms_norm(x, l0.post_norm, plain.rms_norm_eps))
        x, _ = pl.decoder_block(plain, l1, x, torch.arange(len(ids)))
        return pl.output_head(plain, x)

    rng = random.Random(12)
    a, b = H.random_ids(rng, 30, cfg.vocab_size), H.random_ids(rng, 21, cfg.vocab_size)
    want_a, want_b = plain_forward(a), plain_forward(b)
    sa, sb = cache.acquire_slot(), cache.acquire_slot()
    got_a = [runner.step([StepEntry(sa, a[:11], list(range(11)))]).float().cpu().clone()]
    mix = runner.step([StepEntry(sa, a[11:13], [0, 1]), StepEntry(sb, b[:20], list(range(20)))]).float().cpu().clone()
    got_a.append(mix[:2])
    got_b = [mix[2:]]
    both = runner.step([StepEntry(sb, b[20:], [0]), StepEntry(sa, a[13:], list(range(17)))]).float().cpu().clone()
    got_b.append(both[:1])
    got_a.append(both[1:])
    got_a, got_b = torch.cat(got_a), torch.cat(got_b)
    for p in range(30):
        assert H.row_error(got_a[p], want_a[p]) < 2e-5, p
    for p in range(21):
        assert H.row_error(got_b[p], want_b[p]) < 2e-5, p
    # a new request in a used slot starts from a zeroed state
    cache.release_slot(sa)
    sc = cache.acquire_slot()
    assert sc == sa
    again = runner.step([StepEntry(sc, a, list(range(30)))]).float().cpu()
    assert H.row_error(again[29], want_a[29]) < 2e-5


def test_toy_position_encoding_and_routed_feed_forward_are_registered_built_and_stepped():
    """Two more toy parts defined here, with no change to the framework's files: a position
    encoding with a step of its own (it scales q by a function of the position and shifts k along a
    learned direction, instead of rotating), and a feed-forward that routes every token to one of two
    small experts.  Layer 0 uses both, layer 1 is the plain Llama layer; whole prompts and cut ones
    against the same model written out plainly."""
    import bare_cuda_4gib_b200.models  # noqa: F401
    from bare_cuda_4gib_b200.config import LlamaConfig
    from bare_cuda_4gib_b200.engine.model import expected_weights
    from bare_cuda_4gib_b200.engine.step import StepEntry
    from bare_cuda_4gib_b200.kernels.lib import Partials
    from bare_cuda_4gib_b200.models.llama import llama_spec
    from bare_cuda_4gib_b200.parts import Part, PartSpec, register_feed_forward, register_position
    from bare_cuda_4gib_b200.weights import random_tensors

    @register_position("toy_scale_and_shift")
    class ScaleAndShift(Part):
        def local_weights(self):
            return {"direction": ((self.params["head_dim"],), "norm")}

        def fused_rotation(self):
            return None                       # the attention kernels rotate nothing

        def apply(self, ctx, q, k):
            pos = ctx.positions[: q.shape[0]].to(torch.float32)
            q.mul_((1.0 / (1.0 + self.params["rate"] * pos)).to(q.dtype)[:, None, None])
            k.add_((torch.sin(pos)[:, None, None] * self.tensors["direction"].float()[None, None, :]).to(k.dtype))

    @register_feed_forward("toy_two_experts")
    class TwoExperts(Part):
        def local_weights(self):
            h, i = self.params["hidden"], self.params["inner"]
            return {"router": ((2, h), "matrix"), "w_in": ((2 * i, h), "matrix"), "w_out": ((2 * h, i), "matrix")}

        def forward(self, ctx, h):
            hf = h.float()
            i, hidden = self.params["inner"], self.params["hidden"]
            choice = (hf @ self.tensors["router"].float().t()).argmax(-1)          # float32 router logits, top 1
            outs = []
            for e in range(2):
                w_in = self.tensors["w_in"].float()[e * i: (e + 1) * i]
                w_out = self.tensors["w_out"].float()[e * hidden: (e + 1) * hidden]
                outs.append(torch.relu(hf @ w_in.t()) @ w_out.t())
            return Partials(torch.where((choice == 0)[:, None], outs[0], outs[1]).contiguous())

    cfg = LlamaConfig.from_dict(H.TINY_A)
    spec = llama_spec(cfg)
    rate, inner = 0.05, 40
    spec.layers[0].mixer.params["position"] = PartSpec("toy_scale_and_shift", {"head_dim": cfg.head_dim, "rate": rate},
                                                       {"direction": "model.layers.0.toy.direction"})
    spec.layers[0].ffn = PartSpec("toy_two_experts", {"hidden": cfg.hidden_size, "inner": inner},
                                  {"router": "model.layers.0.toy.router", "w_in": "model.layers.0.toy.w_in",
                                   "w_out": "model.layers.0.toy.w_out"})
    expected, model = expected_weights(spec)
    assert "model.layers.0.toy.router" in expected and "model.layers.0.mlp.gate_proj.weight" not in expected
    tensors = {k: v.to("cuda", torch.float32) for k, v in random_tensors(expected, seed=9).items()}
    tensors["model.layers.0.toy.router"] *= 30.0        # clear choices: no token sits on the fence between experts
    model.bind(tensors, torch.float32, "cuda")
    runner, cache = _runner(model, 16, 64)

    t64 = {k: v.double().cpu() for k, v in tensors.items()}
    plain = pl.PlainModel(cfg.vocab_size, cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads,
                          cfg.head_dim, cfg.intermediate_size, cfg.rope_theta, cfg.rms_norm_eps,
                          t64["model.embed_tokens.weight"], t64["model.norm.weight"], t64["lm_head.weight"])
    g0 = lambda n: t64["model.layers.0." + n]
    g1 = lambda n: t64["model.layers.1." + n]
    l1 = pl.PlainLayer(g1("input_layernorm.weight"), g1("self_attn.q_proj.weight"), g1("self_attn.k_proj.weight"),
                       g1("self_attn.v_proj.weight"), g1("self_attn.o_proj.weight"), g1("post_attention_layernorm.weight"),
                       g1("mlp.gate_proj.weight"), g1("mlp.up_proj.weight"), g1("mlp.down_proj.weight"))

    def plain_forward(ids):
        n, nh, nkv, d = len(ids), cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        pos = torch.arange(n, dtype=F64)
        x = pl.embedding(plain.embed, torch.tensor(ids))
        h = pl.rms_norm(x, g0("input_layernorm.weight"), plain.rms_norm_eps)
        q = pl.linear(h, g0("self_attn.q_proj.weight")).view(n, nh, d)
        k = pl.linear(h, g0("self_attn.k_proj.weight")).view(n, nkv, d)
        v = pl.linear(h, g0("self_attn.v_proj.weight")).view(n, nkv, d)
        q = q / (1.0 + rate * pos.float().double())[:, None, None]
        k = k + torch.sin(pos.float()).double()[:, None, None] * g0("toy.direction")[None, None, :]
        probs = torch.softmax(pl.attention_scores(q, k), dim=-1)
        x = x + pl.linear(pl.attention_values(probs, v).reshape(n, nh * d), g0("self_attn.o_proj.weight"))
        h = pl.rms_norm(x, g0("post_attention_layernorm.weight"), plain.rms_norm_eps)
        choice = (h @ g0("toy.router").t()).argmax(-1)
        outs = [torch.relu(h @ g0("toy.w_in")[e * inner: (e + 1) * inner].t())
                @ g0("toy.w_out")[e * cfg.hidden_size: (e + 1) * cfg.hidden_size].t() for e in range(2)]
        x = x + torch.where((choice == 0)[:, None], outs[0], outs[1])
        x, _ = pl.decoder_block(plain, l1, x, torch.arange(n))
        return pl.output_head(plain, x), choice

    rng = random.Random(4)
    a, b = H.random_ids(rng, 33, cfg.vocab_size), H.random_ids(rng, 18, cfg.vocab_size)
    (want_a, choice_a), (want_b, _) = plain_forward(a), plain_forward(b)
    assert 0 < int(choice_a.sum()) < len(a), "both experts must be used"
    sa, sb = cache.acquire_slot(), cache.acquire_slot()
    got_a = [runner.step([StepEntry(sa, a[:7], list(range(7)))]).float().cpu().clone()]
    mix = runner.step([StepEntry(sb, b[:16], list(range(16))), StepEntry(sa, a[7:9], [0, 1])]).float().cpu().clone()
    got_b, got_a = [mix[:16]], got_a + [mix[16:]]
    for p in range(9, 33):                      # request a goes on token by token beside the rest of b
        entries = [StepEntry(sa, [a[p]], [0])] + ([StepEntry(sb, b[16:], [0, 1])] if p == 9 else [])
        out = runner.step(entries).float().cpu().clone()
        got_a.append(out[:1])
        if p == 9:
            got_b.append(out[1:])
    got_a, got_b = torch.cat(got_a), torch.cat(got_b)
    for p in range(33):
        assert H.row_error(got_a[p], want_a[p]) < 2e-5, p
    for p in range(18):
        assert H.row_error(got_b[p], want_b[p]) < 2e-5, p


# ------------------------------------------------------------------------------ a graph-safe mixer with state, under padded decode steps


def test_graph_safe_stateful_mixer_keeps_live_state_clean_when_a_decode_step_is_padded():
    """A toy mixer whose state lives in the per-request slots and is updated on the device (so its
    steps may be captured as CUDA graphs).  Three requests decode together; the step is padded to
    four rows, captured on its second occurrence and replayed.  The idle row must update the spare
    state row that no request owns: request 0 must get what it gets alone."""
    from bare_cuda_4gib_b200.config import LlamaConfig
    from bare_cuda_4gib_b200.engine.model import expected_weights
    from bare_cuda_4gib_b200.engine.step import StepEntry
    from bare_cuda_4gib_b200.kernels.lib import Partials
    from bare_cuda_4gib_b200.models.llama import llama_spec
    from bare_cuda_4gib_b200.parts import Part, PartSpec, StateRequest, register_mixer
    from bare_cuda_4gib_b200.weights import random_tensors

    @register_mixer("toy_running_mean_on_device")
    class RunningMean(Part):
        """state = decay * state + (1 - decay) * h, row by row in row order, with device-side indices
        only: the host loop runs over the step's row count, which is part of a graph's key."""

        def local_weights(self):
            h = self.params["hidden"]
            return {"out": ((h, h), "matrix")}

        def cache_request(self):
            return None

        def state_request(self):
            return StateRequest((self.params["hidden"],), torch.float32)

        def forward(self, ctx, call, h):
            decay = self.params["decay"]
            out = ctx.ws.get("toy_out", (ctx.n_tokens, self.params["hidden"]), torch.float32)
            slot_of_row = ctx.seq_slot.long()[ctx.row_seq[: ctx.n_tokens].long()]      # device indices
            for r in range(ctx.n_tokens):
                index = slot_of_row[r: r + 1]
                state = call.state.index_select(0, index) * decay + h[r: r + 1].float() * (1.0 - decay)
                call.state.index_copy_(0, index, state)
                out[r: r + 1] = state @ self.tensors["out"].float().t()
            return Partials(out)

    cfg = LlamaConfig.from_dict(H.TINY_A)
    spec = llama_spec(cfg)
    decay = 0.5
    spec.layers[0].mixer = PartSpec("toy_running_mean_on_device", {"hidden": cfg.hidden_size, "decay": decay},
                                    {"out": "model.layers.0.toy.out.weight"})
    expected, model = expected_weights(spec)
    tensors = {k: v.to("cuda", torch.float32) for k, v in random_tensors(expected, seed=6).items()}
    model.bind(tensors, torch.float32, "cuda")
    assert model.graph_safe

    def decode(batch_of, steps):
        """Decodes `steps` fixed tokens for the given requests together; returns request 0's logits."""
        runner, cache = _runner(model, 16, 64, max_live=4)
        assert runner.use_cuda_graphs
        slots = [cache.acquire_slot() for _ in batch_of]
        assert slots[0] == 0
        rows = []
        for step in range(steps):
            entries = [StepEntry(s, [(7 * i + 3 * step + 1) % cfg.vocab_size], [0]) for i, s in zip(batch_of, slots)]
            rows.append(runner.step(entries)[0].float().cpu().clone())
        captured = len(runner._graphs)
        state0 = cache.state_of(0)[0].clone()
        spare = cache.state_of(0)[cache.idle_slot].clone()
        return torch.stack(rows), captured, state0, spare

    alone, _, state_alone, spare_alone = decode([0], 6)
    together, captured, state_together, spare_together = decode([0, 1, 2], 6)       # three rows, padded to four
    assert captured >= 1                                      # the padded step ran as a captured graph
    assert float(spare_alone.abs().sum()) == 0.0              # a batch of one is not padded
    assert float(spare_together.abs().sum()) > 0.0            # the idle row did write: into the spare state row
    assert torch.equal(state_alone, state_together)           # ... and nowhere else
    for p in range(6):
        assert H.row_error(together[p], alone[p]) < 2e-5, p
