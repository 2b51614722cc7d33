"""The Nilivik decoder in the library against the plain implementation (``plain_nilivik``): every
mechanism alone, then whole models of several small shapes through the step function, the cache, the
decode state and the entry point. The shapes differ in every size and option: key/value groups of 1 to 3,
key and value heads of different sizes, chunks that are and are not whole pages, head sizes that the
tensor-core kernels take and ones they do not, a loop that starts after the first layer, no loop at all,
a layer without a feed-forward, a pass count of 1 to 3."""
import numpy as np
import pytest
import torch

import dryft_challenge_htn_2026_b200 as dk
import plain_nilivik as plain
from dryft_challenge_htn_2026_b200.cache import Cache, StateRequest
from dryft_challenge_htn_2026_b200.config.specs import DenseMLPSpec, MaskedAttentionSpec, ScalarRMSNormSpec, SinusoidSpec
from dryft_challenge_htn_2026_b200.csrc import api
from dryft_challenge_htn_2026_b200.engine import DecodeLoop, Runner, load_model
from dryft_challenge_htn_2026_b200.engine.batch import build_context
from dryft_challenge_htn_2026_b200.parts import Runtime, build_part
from helpers import random_tokens

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda")
DTYPES = [torch.float32, torch.bfloat16]


def layer_cfg(heads, kv, dim, vdim, chunk, rh, rd, rv, decay, ff, scale=None, ls=0.7, rs=0.6):
    return {"type": "parallel",
            "mixer": {"left": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "mask": {"size": chunk},
                               "scale": scale if scale is not None else dim ** -0.5},
                      "right": {"heads": rh, "dim": rd, "vdim": rv, "decay": decay},
                      "left_scale": ls, "right_scale": rs},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


SHAPES = {
    # groups of 2, value heads smaller than key heads, a chunk that is no whole page, a value size of the linear
    # attention that is no power of two, a layer without feed-forward, a loop that starts at layer 1 and runs 3 times
    "P": dict(architecture="Nilivik", vocab=200, width=64, embedding={"scale": 5.0}, norm={"eps": 1e-5}, logit_softcap=8.0,
              loop={"start": 1, "stop": 3, "times": 3},
              layers=[layer_cfg(4, 2, 32, 16, 24, 2, 16, 24, [0.9, 0.99], 96),
                      layer_cfg(4, 2, 32, 16, 24, 2, 16, 24, [0.5, 0.97], None),
                      layer_cfg(2, 1, 16, 48, 40, 1, 32, 8, [0.95], 72, ls=1.0, rs=0.3)]),
    # no loop, no cap, as many key/value heads as query heads, a chunk of exactly one page, layers that differ
    "Q": dict(architecture="Nilivik", vocab=264, width=96, embedding={"scale": 1.0}, norm={"eps": 3e-6},
              layers=[layer_cfg(3, 3, 16, 48, 64, 3, 32, 32, [0.8, 0.9, 0.999], 128),
                      layer_cfg(6, 2, 16, 16, 7, 2, 48, 16, 0.93, 40)]),
    # head sizes 64 and 128 (what the tensor-core kernels are built for), one pass of the loop's span repeated twice
    "R": dict(architecture="Nilivik", vocab=320, width=128, embedding={"scale": 9.0}, norm={"eps": 1e-5}, logit_softcap=20.0,
              loop={"start": 0, "stop": 1, "times": 2},
              layers=[layer_cfg(2, 1, 64, 64, 100, 2, 64, 64, [0.7, 0.995], 192),
                      layer_cfg(2, 2, 128, 64, 130, 1, 128, 128, [0.98], 160)]),
    # head sizes that no tensor-core kernel takes (20, 10, 24, 12) and an inner size of the output projection (42) and
    # of the feed-forward (52) that is no multiple of 8: the float32-arithmetic kernels and the library's product
    "S": dict(architecture="Nilivik", vocab=136, width=48, embedding={"scale": 2.0}, norm={"eps": 1e-5}, logit_softcap=6.0,
              loop={"start": 0, "stop": 2, "times": 2},
              layers=[layer_cfg(3, 1, 20, 10, 50, 1, 24, 12, [0.96], 52), layer_cfg(3, 3, 20, 10, 33, 1, 24, 12, [0.8], None)]),
}


def make_model(tmp_path, name, seed=0):
    cfg = dk.config_from_dict(SHAPES[name])
    folder = str(tmp_path / f"nilivik{name}_{seed}")
    dk.write_random_model(cfg, folder, seed=seed, dtype=torch.float32, matrix_std=0.08)
    return folder, cfg


def tol(dtype, ref):
    return (2e-4 if dtype in (torch.float32, "float32") else 6e-2) * max(1.0, float(ref.abs().max()))


def rnd(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed), dtype=torch.float64) * scale


def close(got, ref, dtype, what=""):
    err = float((got.double().cpu() - ref.double()).abs().max())
    assert err <= tol(dtype, ref) * 0.5, f"{what}: max error {err} > {tol(dtype, ref) * 0.5}"


# ------------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_scale_and_sinusoid_at_near_and_far_positions(dtype):
    V, W = 50, 72
    table = rnd(V, W, seed=1, scale=0.3).to(dtype)
    pos = [0, 1, 2, 63, 64, 1000, 4097, 250000]
    tok = [3, 7, 7, 49, 0, 11, 12, 13]
    part = build_part(SinusoidSpec(W, 10000.0), Runtime(DEV, dtype))
    h = torch.empty(len(tok), W, dtype=torch.float32, device=DEV)
    a = torch.empty(len(tok), W, dtype=dtype, device=DEV)
    g = torch.full((W,), 1.3, dtype=torch.float32, device=DEV)
    api.embed_position_rmsnorm(torch.tensor(tok, dtype=torch.int32, device=DEV), table.to(DEV), 4.0,
                               torch.tensor(pos, dtype=torch.int32, device=DEV), part.inv_freq, g, 1e-5, h, a)
    ref = table.double()[tok] * 4.0 + plain.sinusoid(pos, W, torch.float64)
    assert float((h.cpu().double() - ref).abs().max()) < 2e-6 * float(ref.abs().max())
    close(a, plain.scalar_norm(ref, 1.3, 1e-5), dtype, "first norm")


@pytest.mark.parametrize("dtype", DTYPES)
def test_scalar_norm_is_one_number_for_all_coordinates(dtype):
    part = build_part(ScalarRMSNormSpec(200, 1e-5), Runtime(DEV, dtype))
    part.bind({"": torch.tensor(0.7, device=DEV)})
    h0, d = rnd(9, 200, seed=2, scale=2.0), rnd(9, 200, seed=3).to(dtype)
    h = h0.float().to(DEV)
    out = part.add_forward(h, d.to(DEV), torch.empty(9, 200, dtype=dtype, device=DEV))
    close(out, plain.scalar_norm(h0.float().double() + d.double(), 0.7, 1e-5), dtype, "scalar norm")


@pytest.mark.parametrize("dtype", DTYPES)
def test_xielu_feed_forward(dtype):
    W, Fw = 64, 104
    part = build_part(DenseMLPSpec(W, Fw, "xielu"), Runtime(DEV, dtype))
    w = {"up": rnd(Fw, W, seed=4, scale=0.3).to(dtype), "down": rnd(W, Fw, seed=5, scale=0.2).to(dtype),
         "act": torch.tensor([0.4, -1.1], dtype=torch.float64)}
    part.bind({"up": w["up"].to(DEV), "down": w["down"].to(DEV), "act": w["act"].float().to(DEV)})
    z = torch.linspace(-9, 9, 64, dtype=torch.float64).to(dtype)
    out = torch.empty(64, dtype=dtype, device=DEV)
    api.xielu(z.to(DEV), out, part.alpha_pos, part.alpha_neg)
    close(out, plain.xielu(z.double(), w["act"][0], w["act"][1]), dtype, "activation")
    for rows in (1, 5, 70, 200):          # the row counts that pick the library's different products
        a = rnd(rows, W, seed=6).to(dtype)
        got = part.forward(None, a.to(DEV))
        got = got.sum(dtype) if isinstance(got, api.Partial) else got
        close(got, plain.dense_ff(a.double(), {k: v.double() for k, v in w.items()}), dtype, f"feed-forward, {rows} rows")


def attention_case(dtype, H, G, D, Dv, chunk, window, lens_steps, bias=True, sink=True, gate=True, plant=None, seed=0):
    """Runs the masked-attention part's ``mix`` (the cache write and whichever attention kernel the part picks for
    the step) over one sequence cut into the steps ``lens_steps`` (and a second sequence beside it, so that rows
    of two sequences share a step) and compares every row with the plain attention over the whole sequence. ``plant`` = (query position, key position, strength):
    that key is made the query's direction, so that its score stands out among all others."""
    T = sum(lens_steps)
    q, k, v = rnd(T, H, D, seed=seed), rnd(T, G, D, seed=seed + 1), rnd(T, G, Dv, seed=seed + 2)
    if plant:
        qi, kj, strength = plant
        k[kj] = strength * q[qi, 0] / q[qi, 0].norm()
        v[kj] = 5.0
    gate_rows = rnd(T, H * Dv, seed=seed + 3) if gate else None
    r1 = (0.1 + rnd(H, seed=seed + 4).abs()) if bias else None
    r2 = (0.05 + rnd(H, seed=seed + 5).abs()) if bias else None
    sk = rnd(H, seed=seed + 6) if sink else None
    cast = lambda x: None if x is None else x.to(dtype)
    q, k, v, gate_rows = cast(q), cast(k), cast(v), cast(gate_rows)
    scale = D ** -0.5
    ref = plain.attention_core(q.double(), k.double(), v.double(), scale, chunk, r1, r2, sk, window).reshape(T, H * Dv)
    if gate:
        ref = ref * torch.sigmoid(gate_rows.double())
    ref = 0.8 * ref
    spec = MaskedAttentionSpec(hidden_size=8, num_heads=H, num_kv_heads=G, head_dim=D, v_head_dim=Dv, scale=scale, chunk=chunk,
                               window=window, distance_bias=bias, sink=sink, output_gate=gate)
    part = build_part(spec, Runtime(DEV, dtype))       # the part picks the kernel for the step; its projections are not used
    f32 = lambda x: None if x is None else x.float().to(DEV)
    part.r1, part.r2, part.sink = f32(r1), f32(r2), f32(sk)
    cache = Cache([part.cache_requests()], 64 * 40, 4, DEV)
    kv = cache.views(0)
    other = cache.begin()                      # a second sequence whose rows sit in front of ours in every step
    slot = cache.begin()
    t0 = 0
    for n in lens_steps:
        m = 1 if n == 1 else 3                 # single-token steps are decode steps: one token for every sequence
        ctx = build_context(cache, [(other, [0] * m, []), (slot, [0] * n, [])], DEV, plans=part.step_plans())
        rows = slice(m, m + n)
        # one wide matrix holds q, k, v and the gate side by side, as a fused projection does
        wide = torch.zeros(m + n, part.n_in + 8, dtype=dtype, device=DEV)
        c0, c1, c2 = H * D, H * D + G * D, H * D + G * D + G * Dv
        wide[rows, :c0] = q[t0:t0 + n].reshape(n, -1).to(DEV)
        wide[rows, c0:c1] = k[t0:t0 + n].reshape(n, -1).to(DEV)
        wide[rows, c1:c2] = v[t0:t0 + n].reshape(n, -1).to(DEV)
        if gate:
            wide[rows, c2:c2 + H * Dv] = gate_rows[t0:t0 + n].to(DEV)
        out = torch.empty(m + n, H * Dv + 8, dtype=dtype, device=DEV)
        part.mix(ctx, kv, wide[:, :part.n_in], out[:, :H * Dv], 0.8)
        close(out[rows, :H * Dv], ref[t0:t0 + n], dtype, f"attention rows {t0}..{t0 + n}")
        cache.commit(other, m)
        cache.commit(slot, n)
        t0 += n
    return cache, slot


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,D,Dv,chunk,window", [(4, 2, 32, 16, 24, None), (3, 3, 16, 48, 64, None), (2, 1, 64, 64, 100, None),
                                                   (2, 1, 80, 80, 50, 20), (6, 2, 128, 64, None, 70), (1, 1, 8, 8, 1, None)])
def test_masked_attention_in_prompts_portions_and_single_tokens(dtype, H, G, D, Dv, chunk, window):
    attention_case(dtype, H, G, D, Dv, chunk, window, [150, 1, 1, 37, 2, 1, 1, 1, 9])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("options", [dict(bias=False, sink=False, gate=False), dict(bias=True, sink=False, gate=False),
                                     dict(bias=False, sink=True, gate=False), dict(bias=False, sink=False, gate=True)])
def test_masked_attention_options_one_at_a_time(dtype, options):
    attention_case(dtype, 4, 2, 32, 32, 48, None, [70, 1, 5], **options)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("where", ["prompt", "decoded"])
@pytest.mark.parametrize("edge", ["first of the chunk", "last before the chunk", "far inside a long chunk", "page border"])
def test_a_planted_key_shows_just_inside_and_is_hidden_just_outside(dtype, where, edge):
    """One key carries a score far above all others and a value of 5: a query that may see it returns
    about 5 * its gate, one that may not returns the ordinary mixture. The plain implementation decides
    which; the planted score makes a mask that is one position off change the output by whole units."""
    chunk = {"first of the chunk": 96, "last before the chunk": 96, "far inside a long chunk": 700, "page border": 128}[edge]
    qi = {"first of the chunk": 200, "last before the chunk": 200, "far inside a long chunk": 690, "page border": 200}[edge]
    kj = {"first of the chunk": 192, "last before the chunk": 191, "far inside a long chunk": 3, "page border": 128}[edge]
    steps = [qi + 6] if where == "prompt" else [qi - 2, 1, 1, 1, 1, 1, 1, 1, 1]
    attention_case(dtype, 2, 1, 32, 32, chunk, None, steps, bias=False, plant=(qi, kj, 60.0), seed=11)


def test_chunked_cache_gives_pages_back_and_takes_them_again():
    cache, slot = attention_case(torch.float32, 2, 1, 16, 16, 70, None, [300, 1, 1, 50])
    g = cache.groups[0]
    held = [p for p in g.pages[slot] if p >= 0]
    assert len(held) == len(g.pages[slot]) - (352 // 70 * 70) // 64        # pages wholly before the current chunk are gone
    free = g.pool.n_free
    cache.end(slot)
    assert g.pool.n_free == free + len(held)
    # the next sequences get those pages and slots: their results must not see what was left there
    attention_case(torch.float32, 2, 1, 16, 16, 70, None, [130, 1, 1], seed=5)


def linear_attention_case(dtype, H, D, Dv, decay, lens_steps, seed=0, scale_k=1.0):
    T = sum(lens_steps)
    q, k, v = (rnd(T, H * D, seed=seed), rnd(T, H * D, seed=seed + 1, scale=scale_k), rnd(T, H * Dv, seed=seed + 2))
    q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
    silu = torch.nn.functional.silu
    ref, last = plain.decay_recurrence(silu(q.double()).view(T, H, D), silu(k.double()).view(T, H, D),
                                       silu(v.double()).view(T, H, Dv), decay)
    cache = Cache([[StateRequest((H, D, Dv), torch.float32)]], 64 * 40, 4, DEV)
    state = cache.views(0)[0].state
    state.fill_(7.0)                            # whatever an earlier sequence left: begin() must clear the slot
    other, slot = cache.begin(), cache.begin()
    dec = torch.tensor(decay, dtype=torch.float32, device=DEV)
    t0 = 0
    for n in lens_steps:
        ctx = build_context(cache, [(other, [0] * 2, []), (slot, [0] * n, [])], DEV)
        wide = torch.zeros(2 + n, 2 * H * D + H * Dv + 8, dtype=dtype, device=DEV)
        wide[2:, :H * D] = q[t0:t0 + n].to(DEV)
        wide[2:, H * D:2 * H * D] = k[t0:t0 + n].to(DEV)
        wide[2:, 2 * H * D:2 * H * D + H * Dv] = v[t0:t0 + n].to(DEV)
        out = torch.empty(2 + n, H * Dv, dtype=torch.float32, device=DEV)
        api.linear_attention(wide[:, :H * D], wide[:, H * D:2 * H * D], wide[:, 2 * H * D:2 * H * D + H * Dv], out, state,
                             ctx.cu_q, ctx.seq_pos0, ctx.seq_slot, dec, ctx.n_seq, H, D, Dv, int(ctx.host["lens"].max()))
        got = out[2:].view(n, H, Dv)
        close(got, ref[t0:t0 + n], dtype, f"linear attention rows {t0}..{t0 + n}")
        cache.commit(other, 2)
        cache.commit(slot, n)
        t0 += n
    close(state[slot], last, dtype, "state after the last step")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,D,Dv,decay", [(2, 16, 24, [0.9, 0.99]), (4, 32, 64, [0.55, 0.85, 0.95, 0.9999]), (1, 32, 8, [0.95]),
                                          (2, 64, 64, [0.7, 0.995]), (1, 128, 128, [0.98]), (3, 48, 16, [1.0, 0.5, 0.2])])
def test_linear_attention_in_prompts_portions_and_single_tokens(dtype, H, D, Dv, decay):
    linear_attention_case(dtype, H, D, Dv, decay, [150, 1, 1, 37, 2, 1, 64, 65, 1])


@pytest.mark.parametrize("dtype", DTYPES)
def test_linear_attention_keeps_a_far_token_under_a_slow_decay(dtype):
    """Decay 0.9995 over 900 tokens keeps 64 % of the first token's outer product: with the keys of the
    first tokens scaled up, a state that is dropped or restarted anywhere on the way shows in every later row."""
    linear_attention_case(dtype, 1, 32, 32, [0.9995], [600, 200, 1, 1, 98, 1], seed=3)


@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_and_gate_over_all_heads_together(dtype):
    n = 3 * 24
    o, w, g = rnd(11, n, seed=1, scale=30.0), 1 + 0.1 * rnd(n, seed=2), rnd(11, n, seed=3).to(dtype)
    out = torch.empty(11, n + 8, dtype=dtype, device=DEV)
    wide_gate = torch.zeros(11, n + 16, dtype=dtype, device=DEV)
    wide_gate[:, 8:8 + n] = g.to(DEV)
    api.norm_gate(o.float().to(DEV), w.float().to(DEV), 1e-5, wide_gate[:, 8:8 + n], 0.5, out[:, :n])
    ref = 0.5 * plain.weighted_norm(o.float().double(), w.float().double(), 1e-5) * torch.sigmoid(g.double())
    close(out[:, :n], ref, dtype, "norm and gate")


# ----------------------------------------------------------------------------------------- whole models
def plain_logits(folder, tokens):
    cfg, t = plain.read_model(folder, torch.float64)
    return plain.forward(cfg, t, tokens)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "Q", "R", "S"])
def test_whole_prompts_portions_batches_and_reused_slots(tmp_path, name, dtype):
    folder, cfg = make_model(tmp_path, name)
    model = load_model(folder, dtype)
    runner = Runner(model, 64 * 24, 6)
    lens = [1, 23, 131, 200]
    seqs = [random_tokens(cfg.vocab, n, 40 + i) for i, n in enumerate(lens)]
    ref = [plain_logits(folder, s) for s in seqs]

    def check(out, pairs, what):
        out = out.cpu().double()
        for row, (i, p) in enumerate(pairs):
            err = float((out[row] - ref[i][p]).abs().max())
            assert err <= tol(dtype, ref[i]), f"{name} {what}: sequence {i} position {p}: {err}"

    for round_ in range(2):        # the second round runs on the slots and pages the first gave back
        # each alone, whole
        for i, s in enumerate(seqs):
            slot = runner.begin()
            want = sorted({0, len(s) // 2, len(s) - 1})
            check(runner.step([(slot, s, want)]), [(i, p) for p in want], "alone")
            runner.end(slot)
        # together: a ragged batch of prompts cut short, then one token each, shorter ones ending earlier
        cut = [1, 17, 100, 130]
        slots = [runner.begin() for _ in seqs]
        check(runner.step([(sl, s[:c], [c - 1]) for sl, s, c in zip(slots, seqs, cut)]), [(i, c - 1) for i, c in enumerate(cut)],
              "batch of prompts")
        live = [i for i in range(4) if cut[i] < lens[i]]
        k = 0
        while live and k < 40:
            out = runner.step([(slots[i], [seqs[i][cut[i] + k]], [0]) for i in live])
            check(out, [(i, cut[i] + k) for i in live], f"decode step {k}")
            k += 1
            for i in [i for i in live if cut[i] + k >= lens[i]]:
                runner.end(slots[i])
                slots[i] = None
            live = [i for i in live if cut[i] + k < lens[i]]
        for sl in slots:
            if sl is not None:
                runner.end(sl)
        # portions of several sizes, down to two tokens and one
        s, i = seqs[3], 3
        slot = runner.begin()
        at = 0
        for n in [64, 2, 31, 1, 2, 70, 30]:
            check(runner.step([(slot, s[at:at + n], [0, n - 1])]), [(i, at), (i, at + n - 1)], f"portion of {n} at {at}")
            at += n
        runner.end(slot)
    assert runner.cache.slots.n_live == 0 and all(f == runner.cache.num_pages for f in runner.cache.pages_free())


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_through_the_decode_state_and_its_graph(tmp_path, dtype):
    folder, cfg = make_model(tmp_path, "P", seed=3)
    model = load_model(folder, dtype)
    seqs = [random_tokens(cfg.vocab, n, 60 + i) for i, n in enumerate([150, 90])]
    ref = [plain_logits(folder, s) for s in seqs]
    for use_graph in (False, True):
        runner = Runner(model, 64 * 12, 4)
        loop = DecodeLoop(runner, use_graph=use_graph)
        slots = [runner.begin() for _ in seqs]
        cut = [30, 5]
        runner.step([(sl, s[:c], []) for sl, s, c in zip(slots, seqs, cut)])
        for k in range(85):                          # across page borders and several chunks of 24 and 40 positions
            out = loop.forced_step([(sl, [s[c + k]], [0]) for sl, s, c in zip(slots, seqs, cut)]).cpu().double()
            for i in range(2):
                err = float((out[i] - ref[i][cut[i] + k]).abs().max())
                assert err <= tol(dtype, ref[i]), f"graph={use_graph} step {k} sequence {i}: {err}"
        for sl in slots:
            runner.end(sl)
    api.gemm_tc_check()


@pytest.mark.parametrize("name", ["P", "R"])
def test_greedy_generation_through_the_entry_point(tmp_path, name):
    folder, cfg = make_model(tmp_path, name, seed=5)
    pcfg, t = plain.read_model(folder, torch.float64)
    prompts = [random_tokens(cfg.vocab, n, 80 + i) for i, n in enumerate([3, 40, 77])]
    n_new = 30
    for dtype in DTYPES:
        eng = dk.Engine(folder, dtype=dtype)
        steps = list(eng.generate(prompts, n_new))
        again = list(dk.Engine(folder, dtype=dtype, use_graph=False, max_prefill_tokens=16).generate(prompts, n_new))
        for i, p in enumerate(prompts):
            emitted = [s[i] for s in steps]
            logits = plain.forward(pcfg, t, p + emitted[:-1])[len(p) - 1:]
            gap = float((logits.max(-1).values - logits.gather(1, torch.tensor(emitted).view(-1, 1)).squeeze(1)).max())
            assert gap <= (1e-4 if dtype == torch.float32 else 0.12 * max(1.0, float(logits.abs().max()))), (name, dtype, i, gap)
            if dtype == torch.float32:               # prompts cut into portions of 16, plain launches: the same tokens
                assert emitted == [s[i] for s in again]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_of_a_ragged_schedule(tmp_path, dtype):
    folder, cfg = make_model(tmp_path, "Q", seed=7)
    seqs = {"a": random_tokens(cfg.vocab, 140, 1), "b": random_tokens(cfg.vocab, 9, 2), "c": random_tokens(cfg.vocab, 66, 3)}
    ref = {k: plain_logits(folder, s) for k, s in seqs.items()}
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": seqs["a"][:130], "want": [0, 63, 64, 129]},
                                     {"id": "b", "tokens": seqs["b"][:5], "want": [4]},
                                     {"id": "c", "tokens": seqs["c"][:60], "want": []}], "end": []}]
    for k in range(10):
        ent = [{"id": "a", "tokens": [seqs["a"][130 + k]], "want": [0]}]
        if 5 + k < 9:
            ent.append({"id": "b", "tokens": [seqs["b"][5 + k]], "want": [0]})
        if 60 + k < 66:
            ent.append({"id": "c", "tokens": [seqs["c"][60 + k]], "want": [0] if k % 2 else []})
        steps.append({"step": k + 1, "entries": ent, "end": [i for i, n in (("b", 9), ("c", 66), ("a", 140)) if
                                                             any(e["id"] == i for e in ent) and {"a": 130, "b": 5, "c": 60}[i] + k + 1 == n]})
    with open(f"{folder}/config.json") as f:
        import json
        vocab = json.load(f)["vocab"]
    import os
    import subprocess
    import sys
    from helpers import ROOT
    out_dir = str(tmp_path / "out")
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
                           "--out", out_dir, "--max-tokens", "512"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                          capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-3000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done ")] == [f"done {s['step']}" for s in steps]
    at = {"a": 0, "b": 0, "c": 0}
    for s in steps:
        rows = []
        for e in s["entries"]:
            rows += [(e["id"], at[e["id"]] + w) for w in e["want"]]
            at[e["id"]] += len(e["tokens"])
        if rows:
            got = torch.from_numpy(np.fromfile(os.path.join(out_dir, f"{s['step']}.f32"), dtype="<f4").reshape(len(rows), vocab))
            for r, (i, p) in enumerate(rows):
                assert float((got[r].double() - ref[i][p]).abs().max()) <= tol(dtype, ref[i]), (s["step"], i, p)


def test_command_line_generates_with_a_nilivik_model(tmp_path):
    """The command line as a user runs it: random weights from a config.json of this design, the tokens it
    prints against the plain implementation's greedy tokens, then the saved folder in bfloat16 with JSON records."""
    import json
    import os
    import subprocess
    import sys
    from dryft_challenge_htn_2026_b200.cli import random_prompts
    from helpers import ROOT

    def run_cli(*args):
        env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
        return subprocess.run([sys.executable, "-m", "dryft_challenge_htn_2026_b200.cli", *args], capture_output=True,
                              text=True, env=env, cwd=str(ROOT), timeout=900)

    cfg = dk.config_from_dict(SHAPES["P"])
    cfg.save(str(tmp_path))
    model_dir = str(tmp_path / "model")
    r = run_cli("--random-weights", str(tmp_path / "config.json"), "--save-model", model_dir, "--seed", "3", "--dtype", "float32",
                "--shapes", "2,30,6", "--samples", "1", "--print-tokens")
    assert r.returncode == 0, r.stdout + r.stderr
    lines = [l for l in r.stdout.splitlines() if l.startswith("tokens 2,30,6 seq ")]
    assert len(lines) == 2
    pcfg, t = plain.read_model(model_dir, torch.float64)
    prompts = random_prompts(2, 30, 1, cfg.vocab, False)
    for i, line in enumerate(lines):
        emitted = [int(x) for x in line.split(":")[1].split()]
        if emitted != plain.greedy(pcfg, t, prompts[i], 6):                 # a near-tie may flip: then the gap is rounding-small
            logits = plain.forward(pcfg, t, prompts[i] + emitted[:-1])[len(prompts[i]) - 1:]
            gap = float((logits.max(-1).values - logits.gather(1, torch.tensor(emitted).view(-1, 1)).squeeze(1)).max())
            assert gap < 1e-3, (emitted, gap)
    r = run_cli("--model", model_dir, "--shapes", "3,70,5", "--samples", "1", "--ragged", "--json")
    assert r.returncode == 0, r.stdout + r.stderr
    records = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")]
    assert [x["shape"] for x in records] == ["3,70,5"] and records[0]["tok_s"] > 0
