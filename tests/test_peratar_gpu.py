"""The Peratar design in the engine against the plain implementation in ``plain_peratar``.

First each mechanism's kernel alone (norms, the gated join with the depth mix, the activation,
the soft cap, the preparation of latent attention, the per-head products), then whole models
through trace replay: whole prompts, the last tokens decoded one by one, portions down to two
tokens, mixed batches in a pool so small that pages and slots are used again, long decoding
across many page borders, the first tokens of a sequence, a needle far back that the attention
must find, and greedy generation through the engine's entry point and scheduler.
"""
import math

import numpy as np
import pytest
import torch

import peratar_configs as pc
import plain_peratar as plain
from helpers import check_logits as _check_logits, random_prompts

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def check_logits(got, want, dtype, what):
    """The tests' weights sharpen the softmax (scores of +-10), which multiplies what the rounding
    of queries and keys to 8 bits does to the weights: bfloat16 gets twice the usual allowance.
    float32, which runs the same layouts, pages and schedules, keeps 2e-5."""
    _check_logits(got, want, dtype, what, bf16_tolerance=6e-2, bf16_min_cosine=0.997)


def close(got, want, dtype, what, scale=None):
    got, want = got.double().cpu(), want.double().cpu()
    scale = float(want.abs().max()) if scale is None else scale
    tol = (3e-6 if dtype == "float32" else 1.2e-2) * max(scale, 1e-6)
    err = float((got - want).abs().max())
    assert err <= tol, f"{what} ({dtype}): max error {err:.3e}, allowed {tol:.3e}"


# ------------------------------------------------------------------------------------ kernels
@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("width", [40, 96, 1000, 9000])
def test_layer_norm_rows(dtype, width):
    from velox_b200.ops import kernels

    dt = DTYPES[dtype]
    gen = torch.Generator().manual_seed(width)
    resid = (torch.randn(7, width, generator=gen) * 3 + 1.5).cuda()
    delta = torch.randn(7, width, generator=gen).to(dt).cuda()
    weight = (1 + 0.2 * torch.randn(width, generator=gen)).cuda()
    rows = torch.tensor([5, 0, 3], dtype=torch.int32).cuda()
    out = torch.zeros(3, width, dtype=dt).cuda()
    before = resid.clone()
    kernels.norm_rows(resid, delta, weight, 1e-5, True, out, 3, rows, write_resid=False)
    assert torch.equal(resid, before)
    want = plain.layer_norm((before.double() + delta.double())[rows.long()], weight.double(), 1e-5)
    close(out, want, dtype, "layer norm of selected rows")
    out2 = torch.zeros(7, width, dtype=dt).cuda()
    kernels.norm_rows(resid, None, weight, 1e-5, False, out2, 7)
    close(out2, plain.rms_norm(before.double(), weight.double(), 1e-5), dtype, "rms norm through the same kernel")


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("width,terms", [(96, 0), (96, 1), (200, 4), (9000, 3)])
def test_gated_join_and_depth_mix(dtype, width, terms):
    from velox_b200.ops import kernels

    dt = DTYPES[dtype]
    gen = torch.Generator().manual_seed(width + terms)
    rows, pitch = 5, width + 24
    wide = torch.randn(rows, pitch, generator=gen).to(dt).cuda()       # delta in columns 8 ..
    gates = (2 * torch.randn(rows, pitch, generator=gen)).to(dt).cuda()  # gate in columns 16 ..
    delta, gate = wide[:, 8 : 8 + width], gates[:, 16 : 16 + width]
    weight = (1 + 0.2 * torch.randn(width, generator=gen)).cuda()
    store = torch.randn(6, rows, width, generator=gen).cuda()
    mix_w = torch.randn(max(terms, 1), generator=gen).cuda()
    x_in = store[terms - 1].clone() if terms > 1 else torch.randn(rows, width, generator=gen).cuda()
    x_out = store[max(terms - 1, 0)]
    mix_out = store[terms] if terms else None
    lowp = torch.zeros(rows, width, dtype=dt).cuda()
    earlier = store[: max(terms - 1, 0)].clone().double()
    kernels.gated_norm_add(x_in, x_out, delta, gate, weight, 1e-5, True, rows, lowp_out=lowp,
                           history=store if terms else None, mix_weights=mix_w[:terms] if terms else None,
                           mix_out=mix_out)
    y = delta.double() * torch.sigmoid(gate.double())
    x = x_in.double() + plain.layer_norm(y, weight.double(), 1e-5)
    close(x_out, x, dtype, "stream after the join")
    going = x
    if terms:
        going = plain.depth_mix(list(earlier) + [x], mix_w[:terms].double())
        close(mix_out, going, dtype, "depth mix")
    close(lowp, going, dtype, "outgoing rows in the compute dtype")
    # without a gate
    kernels.gated_norm_add(x_in, x_out, delta, None, weight, 1e-5, False, rows)
    close(x_out, x_in.double() + plain.rms_norm(delta.double(), weight.double(), 1e-5), dtype, "ungated rms join")
    # the result as float32 sums with a bias still to add; the rows read are handed back empty
    sums = torch.randn(rows + 2, width, generator=gen).cuda()
    bias = torch.randn(width, generator=gen).cuda()
    kept = sums.clone()
    kernels.gated_norm_add(x_in, x_out, None, gate, weight, 1e-5, True, rows, sums=sums, sums_bias=bias, compute_dtype=dt)
    y = (kept[:rows].double() + bias.double()) * torch.sigmoid(gate.double())
    close(x_out, x_in.double() + plain.layer_norm(y, weight.double(), 1e-5), dtype, "join of float32 sums")
    assert torch.all(sums[:rows] == 0) and torch.equal(sums[rows:], kept[rows:])


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_xielu_and_softcap(dtype):
    from velox_b200.ops import kernels

    dt = DTYPES[dtype]
    z = torch.cat([torch.linspace(-9, 9, 301), torch.tensor([0.0, -1e-4, 1e-4, -30.0])]).repeat(3, 1)
    buf = torch.zeros(3, z.shape[1] + 5, dtype=dt).cuda()
    buf[:, 5:] = z.to(dt)
    out = torch.zeros(3, z.shape[1], dtype=dt).cuda()
    p, q = 0.7, -1.3
    kernels.xielu(buf[:, 5:], out, 3, plain.softplus(p), 0.5 + plain.softplus(q))
    close(out, plain.xielu(buf[:, 5:].double().cpu(), p, q), dtype, "xielu")
    logits = (40 * torch.randn(4, 77)).cuda()
    want = 11.0 * torch.tanh(logits.double() / 11.0)
    kernels.softcap(logits, 4, 11.0)
    close(logits, want, "float32", "soft cap")


@pytest.mark.parametrize("tokens,side,inner,width", [(1, 0, 72, 64), (9, 64, 200, 64), (100, 128, 330, 128), (256, 8, 64, 256)])
def test_projection_with_activation_in_its_epilogue(tokens, side, inner, width):
    """The tensor-core projection that writes its first columns as they are and the others through
    the activation into a second buffer, against the two steps made plainly."""
    from velox_b200.ops import kernels

    gen = torch.Generator().manual_seed(tokens + inner)
    x = torch.randn(tokens + 3, width, generator=gen).to(torch.bfloat16).cuda()
    w = (2 * torch.randn(side + inner, width, generator=gen) / width ** 0.5).to(torch.bfloat16).cuda()
    bias = torch.randn(side + inner, generator=gen).cuda()
    out = torch.zeros(tokens + 3, side + inner + 8, dtype=torch.bfloat16).cuda()
    act = torch.zeros(tokens + 3, inner, dtype=torch.bfloat16).cuda()
    status = torch.zeros(4, dtype=torch.int32).cuda()
    p, q = -0.2, 0.9
    assert kernels.gemm_bf16_xielu(x, w, bias, out, act, side, plain.softplus(p), 0.5 + plain.softplus(q), tokens, status)
    assert int(status[0]) == 0
    full = x[:tokens].double() @ w.double().T + bias.double()
    if side:
        close(out[:tokens, :side], full[:, :side], "bfloat16", "columns that pass")
    close(act[:tokens], plain.xielu(full[:, side:].cpu(), p, q), "bfloat16", "activated columns")
    assert torch.all(act[tokens:] == 0) and torch.all(out[:, side:] == 0)


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("heads,dim,rot,rot_dims,rank", [(3, 16, 8, 8, 40), (1, 8, 12, 8, 20), (5, 24, 6, 6, 33)])
def test_latent_prepare(dtype, heads, dim, rot, rot_dims, rank):
    from velox_b200.ops import kernels
    from velox_b200.parts.registry import part_class

    dt = DTYPES[dtype]
    dev = torch.device("cuda")
    gen = torch.Generator().manual_seed(heads * 100 + rank)
    T, page, pages = 9, 4, 6
    padded = -(-(rank + rot) // 16) * 16
    q_width = heads * (dim + rot)
    proj = torch.randn(T, q_width + rank + rot + 3, generator=gen).to(dt).cuda()
    positions = torch.tensor([0, 1, 2, 3, 700, 701, 5, 0, 1023], dtype=torch.int32).cuda()
    slots = torch.tensor([4, 5, 6, 7, 20, 21, 9, -1, 13], dtype=torch.int32).cuda()
    rope = part_class("position", "rotary_interleaved")({"rotary_dim": rot_dims, "base": 5000.0, "max_position": 1024},
                                                        {}, dt, dev)
    weight = (1 + 0.3 * torch.randn(rank, generator=gen)).cuda()
    cache = torch.full((pages, page, 1, padded), 7.0, dtype=dt).cuda()
    queries = torch.full((T, heads, padded), 5.0, dtype=dt).cuda()
    status = torch.zeros(4, dtype=torch.int32).cuda()
    kernels.latent_prepare(proj, 0, q_width, positions, rope.cos, rope.sin, weight, 1e-5, slots, cache, queries, T,
                           heads, dim, rot, rank, status)
    assert int(status[0]) == 0
    p64, pos = proj.double().cpu(), positions.cpu()
    q = p64[:, :q_width].view(T, heads, dim + rot)
    want_q = plain.rotate_pairs(q[..., dim:], pos, 5000.0, rot_dims)
    close(queries[..., rank : rank + rot], want_q, dtype, "rotated query parts")
    assert torch.all(queries[..., rank + rot :] == 0) and torch.all(queries[..., :rank] == 5.0)
    latent = plain.rms_norm(p64[:, q_width : q_width + rank], weight.double().cpu(), 1e-5)
    key = plain.rotate_pairs(p64[:, q_width + rank : q_width + rank + rot], pos, 5000.0, rot_dims)
    flat = cache.view(pages * page, padded)
    for t in range(T):
        s = int(slots[t])
        if s < 0:
            continue
        close(flat[s, :rank], latent[t], dtype, f"latent of token {t}")
        close(flat[s, rank : rank + rot], key[t], dtype, f"key part of token {t}")
        assert torch.all(flat[s, rank + rot :] == 0)
    untouched = sorted(set(range(pages * page)) - {int(s) for s in slots if s >= 0})
    assert torch.all(flat[untouched] == 7.0), "a slot that no token names was written"
    # a slot outside the pool is refused and reported, not written
    bad = slots.clone()
    bad[0] = pages * page
    kernels.latent_prepare(proj, 0, q_width, positions, rope.cos, rope.sin, weight, 1e-5, bad, cache, queries, T,
                           heads, dim, rot, rank, status)
    assert int(status[0]) & 4
    # a layer without a latent of its own rotates its queries and writes nothing
    cache2 = cache.clone()
    kernels.latent_prepare(proj, 0, None, positions, rope.cos, rope.sin, None, 1e-5, None, None, queries, T,
                           heads, dim, rot, rank, status)
    assert torch.equal(cache, cache2)


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("heads,n,k,tokens", [(3, 40, 16, 9), (1, 7, 33, 1), (5, 16, 96, 300)])
def test_headwise_linear(dtype, heads, n, k, tokens):
    from velox_b200.ops import kernels

    dt = DTYPES[dtype]
    gen = torch.Generator().manual_seed(n * k)
    x = torch.randn(tokens, 5 + heads * (k + 3), generator=gen).to(dt).cuda()
    w = (torch.randn(heads, n, k, generator=gen) / k ** 0.5).to(dt).cuda()
    g = torch.randn(tokens, heads + 2, generator=gen).to(dt).cuda()
    out = torch.zeros(tokens, heads * (n + 1) + 4, dtype=dt).cuda()
    kernels.headwise_linear(x, 5, k + 3, w, out, 4, n + 1, tokens, gate=g, gate_offset=2)
    xs = torch.stack([x[:, 5 + h * (k + 3) : 5 + h * (k + 3) + k] for h in range(heads)], 1).double()
    want = torch.einsum("thk,hnk->thn", xs, w.double()) * torch.sigmoid(g[:, 2:].double())[..., None]
    for h in range(heads):
        close(out[:, 4 + h * (n + 1) : 4 + h * (n + 1) + n], want[:, h], dtype, f"head {h}")
    assert torch.all(out[:, :4] == 0)


# ------------------------------------------------------------------------------------ models
CASES = {
    # name -> (config, page size, request lengths, sharpness of the attention: at these values the
    # largest softmax weight of a query is 0.5 to 0.7 on average and scores reach +-20 to 30)
    "small": (pc.SMALL, 4, (5, 11, 17, 60, 100), 2.0),
    "odd": (pc.ODD, 16, (1, 9, 33, 70, 150), 1.5),
    "wide": (pc.WIDE, 64, (130, 3, 65, 300, 64), 3.0),
}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, (cfg, page, lengths, sharp) in CASES.items():
        folder = str(tmp_path_factory.mktemp("peratar_" + name))
        tensors = pc.make_weights(cfg, seed=5 + len(name), sharp=sharp)
        pc.write_folder(folder, cfg, tensors)
        prompts = random_prompts(cfg["vocab"], lengths, seed=31)
        want = [plain.forward_logits(tensors, cfg, p) for p in prompts]
        out[name] = (folder, cfg, page, prompts, want, tensors)
    return out


def make_replayer(folder, dtype, max_tokens, page, **kw):
    from velox_b200.engine.replay import TraceReplayer

    return TraceReplayer(folder, dtype, max_tokens, block_size=page, **kw)


def replay_one(replayer, name, tokens, cuts):
    rows, start = [], 0
    for step, n in enumerate(cuts):
        rec = {"step": step, "entries": [{"id": name, "tokens": tokens[start : start + n], "want": list(range(n))}],
               "end": [name] if start + n == len(tokens) else []}
        rows.append(replayer.run_step(rec))
        start += n
    assert start == len(tokens)
    return np.concatenate(rows, axis=0)


def changing_cuts(total):
    sizes = [7, 2, 16, 3, 2, 5, 33, 2, 9, 64, 4, 2, 21]
    cuts, left, i = [], total, 0
    while left > 0:
        n = min(sizes[i % len(sizes)], left)
        if left - n == 1:
            n = left
        cuts.append(n)
        left -= n
        i += 1
    return cuts


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("case", list(CASES))
def test_whole_then_decode_then_portions(models, case, dtype):
    folder, cfg, page, prompts, want, _ = models[case]
    longest = max(len(p) for p in prompts)
    replayer = make_replayer(folder, dtype, max_tokens=max(256, -(-longest // 64) * 64), page=page)
    for index, (tokens, ref) in enumerate(zip(prompts, want)):
        L = len(tokens)
        whole = replay_one(replayer, f"w{index}", tokens, [L])
        check_logits(whole, ref, dtype, f"{case} request {index} whole")
        tail = min(32, L - 1)
        if tail > 0:
            decoded = replay_one(replayer, f"d{index}", tokens, [L - tail] + [1] * tail)
            check_logits(decoded, ref, dtype, f"{case} request {index} last {tail} one by one")
            if dtype == "float32":
                assert np.array_equal(decoded, whole), "decode differs from the whole prompt in float32"
        if L > 2:
            portions = replay_one(replayer, f"p{index}", tokens, changing_cuts(L))
            check_logits(portions, ref, dtype, f"{case} request {index} in portions")
            if dtype == "float32":
                assert np.array_equal(portions, whole), "portions differ from the whole prompt in float32"
    replayer.cache.assert_consistent()
    assert replayer.cache.num_free_pages() == replayer.cache.num_total_pages
    assert replayer.cache.num_free_slots == replayer.max_live


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("case", ["many_heads", "ragged", "largest_row"])
def test_other_sizes(tmp_path, case, dtype):
    """Sizes at the edges of what the kernels take, one request whole, decoded and in portions."""
    cfg = pc.ALL[case]
    tensors = pc.make_weights(cfg, seed=3, sharp=1.5)
    folder = str(tmp_path / case)
    pc.write_folder(folder, cfg, tensors)
    tokens = random_prompts(cfg["vocab"], [150], seed=1)[0]
    ref = plain.forward_logits(tensors, cfg, tokens)
    replayer = make_replayer(folder, dtype, max_tokens=192, page=16)
    whole = replay_one(replayer, "w", tokens, [150])
    decoded = replay_one(replayer, "d", tokens, [120] + [1] * 30)
    portions = replay_one(replayer, "p", tokens, changing_cuts(150))
    for what, got in (("whole", whole), ("decoded", decoded), ("portions", portions)):
        check_logits(got, ref, dtype, f"{case} {what}")
    if dtype == "float32":
        assert np.array_equal(whole, decoded) and np.array_equal(whole, portions)


def mixed_trace(prompts, rng, max_live=4):
    progress = [0] * len(prompts)
    waiting = list(range(len(prompts)))
    live, steps = [], []
    step = 0
    while waiting or live:
        while waiting and len(live) < max_live:
            live.append(waiting.pop(0))
        entries, ends = [], []
        for r in list(live):
            left = len(prompts[r]) - progress[r]
            if rng.random() < 0.2 and len(live) > 1:
                continue
            decoding = left <= 12 or rng.random() < 0.3
            n = 1 if decoding else min(left, int(rng.choice([2, 3, 5, 8, 13, 30])))
            if left - n == 0:
                ends.append(r)
            entries.append((r, progress[r], n))
            progress[r] += n
        if not entries:
            continue
        steps.append((step, entries, ends))
        for r in ends:
            live.remove(r)
        step += 1
    return steps


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("case", list(CASES))
def test_mixed_batches_with_pages_and_slots_used_again(models, case, dtype):
    folder, cfg, page, prompts, want, _ = models[case]
    order = list(range(len(prompts))) * 2
    seqs = [prompts[i] for i in order]
    steps = mixed_trace(seqs, np.random.default_rng(9))
    need = sum(sorted((-(-len(p) // 64) * 64 for p in prompts), reverse=True)[:4])
    replayer = make_replayer(folder, dtype, max_tokens=need, page=page, max_live=4)
    got = [np.zeros((len(p), cfg["vocab"]), np.float32) for p in seqs]
    slots_used = []
    for step, entries, ends in steps:
        rec = {"step": step, "end": [f"r{r}" for r in ends],
               "entries": [{"id": f"r{r}", "tokens": seqs[r][s : s + n], "want": list(range(n))} for r, s, n in entries]}
        out = replayer.run_step(rec)
        row = 0
        for r, s, n in entries:
            got[r][s : s + n] = out[row : row + n]
            row += n
        slots_used.extend(seq.slot for seq in replayer.live.values())
        replayer.cache.assert_consistent()
    for r, ref_index in enumerate(order):
        check_logits(got[r], want[ref_index], dtype, f"{case} mixed request {r}")
    if dtype == "float32":
        for r in range(len(prompts)):
            assert np.array_equal(got[r], got[r + len(prompts)]), f"request {r}: pages or neighbours changed its logits"
    assert replayer.cache.num_free_pages() == replayer.cache.num_total_pages
    assert set(slots_used) <= set(range(4))


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("case,page", [("small", 4), ("wide", 16)])
def test_long_decode_across_pages_and_split_key_ranges(models, case, page, dtype):
    folder, cfg, _, _, _, tensors = models[case]
    tokens = random_prompts(cfg["vocab"], [420], seed=4)[0]
    ref = plain.forward_logits(tensors, cfg, tokens)
    replayer = make_replayer(folder, dtype, max_tokens=448, page=page,
                             plan_overrides={"min_split_keys": 64, "target_ctas": 4096})
    rows = replay_one(replayer, "long", tokens, [30] + [1] * 390)
    check_logits(rows, ref, dtype, "long decode")


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_long_prompt_whole_and_in_large_portions(models, dtype):
    """Steps above the small-step limit of the projections and attention tiles far from the start."""
    folder, cfg, page, _, _, tensors = models["wide"]
    tokens = random_prompts(cfg["vocab"], [600], seed=14)[0]
    ref = plain.forward_logits(tensors, cfg, tokens)
    replayer = make_replayer(folder, dtype, max_tokens=640, page=page)
    check_logits(replay_one(replayer, "whole", tokens, [600]), ref, dtype, "600 tokens whole")
    check_logits(replay_one(replayer, "parts", tokens, [300, 299, 1]), ref, dtype, "600 tokens as 300 + 299 + 1")


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_first_tokens(models, dtype):
    folder, cfg, page, prompts, want, _ = models["odd"]
    replayer = make_replayer(folder, dtype, max_tokens=64, page=page)
    rows = replay_one(replayer, "f", prompts[3][:6], [1, 1, 2, 2])
    check_logits(rows, want[3][:6], dtype, "first tokens")


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("needle_at", [0, 3, 63, 64, 65, 127, 128, 301])
def test_needle_far_back(tmp_path, dtype, needle_at):
    """One key, at a page border, at the very start or hundreds of tokens back, gets nearly all
    of the softmax weight of the last queries: the first layer's query and shared key part are
    made so that a marker token's key part lines up with the last tokens' queries, unrotated
    (the rotated dims that turn are zeroed for both).  Losing that key changes the logits."""
    cfg = pc.config(64, 90, [
        pc.layer(pc.mixer(2, 8, 8, 16, 24, 1.0, base=100.0, rot_dims=4), 48),
        pc.layer(pc.mixer(2, 8, 8, 16, 24, 1.0, base=100.0, rot_dims=4, kv_from=0), None),
    ], cap=20.0)
    tensors = {k: v.float() for k, v in pc.make_weights(cfg, seed=2, sharp=1.0).items()}
    marker, asker = 7, 11
    for name in ("l0.mix.q", "l1.mix.q"):
        q = tensors[name].view(2, 16, 64)
        q[:, 8:12] = 0                      # the turning dims of the rotated part play no role
        q[:, 12:16] = 0
        q[:, 12] = 6.0 * tensors["embed"][asker] / tensors["embed"][asker].norm()
    dkv = tensors["l0.mix.dkv"]
    dkv[24:28] = 0
    dkv[28:32] = 0
    dkv[28] = 6.0 * tensors["embed"][marker] / tensors["embed"][marker].norm()
    tensors = {k: v.to(torch.bfloat16) for k, v in tensors.items()}
    folder = str(tmp_path / "needle")
    pc.write_folder(folder, cfg, tensors)
    length = 330
    tokens = [t if t not in (marker, asker) else 20 for t in random_prompts(90, [length], seed=needle_at)[0]]
    tokens[needle_at] = marker
    tokens[-3:] = [asker] * 3
    ref = plain.forward_logits(tensors, cfg, tokens)
    without = list(tokens)
    without[needle_at] = 21
    moved = (plain.forward_logits(tensors, cfg, without)[-1] - ref[-1]).abs().max().item()
    assert moved > 0.3, f"the needle does not matter enough for this test ({moved:.3f})"
    replayer = make_replayer(folder, dtype, max_tokens=384, page=64)
    rows = replay_one(replayer, "n", tokens, [length - 3, 1, 2])
    check_logits(rows[-3:], ref[-3:], dtype, f"needle at {needle_at}, decoded")
    rows = replay_one(replayer, "m", tokens, [100, 2, 200, 28])
    check_logits(rows[-3:], ref[-3:], dtype, f"needle at {needle_at}, in portions")


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_layer_streams(models, dtype):
    """The stream after every layer, read back from the block's store of results."""
    folder, cfg, page, prompts, _, tensors = models["odd"]
    tokens = prompts[2]
    _, mixed, results = plain.forward_states(tensors, cfg, tokens)
    replayer = make_replayer(folder, dtype, max_tokens=64, page=page, enable_graphs=False)
    replay_one(replayer, "s", tokens, [len(tokens)])
    store = replayer.runner.workspace._buffers["block.results"]
    # Slot j ends up holding the result X_j (a layer works in place on the mixed rows it was
    # given); the slot after the last result holds the last mix, which the final norm reads.
    wanted = list(results) + [mixed[-1]]
    for index, want in enumerate(wanted):
        got = store[index, : len(tokens)].double().cpu()
        if dtype == "float32":
            # a layer norm of a small sublayer result multiplies the rounding before it
            close(got, want, dtype, f"slot {index} of the store of results", scale=8 * float(want.abs().max()))
        else:
            # single elements behind such a norm can be off by several per cent; the rows are not
            relative = float((got - want).norm() / want.norm())
            assert relative <= 3e-2, f"slot {index} of the store of results: relative error {relative:.3f}"


def test_command_lines_take_the_design(tmp_path, capsys):
    """The benchmark and roofline command lines on the tiny named size of the design."""
    import json

    from velox_b200.cli import benchmark, roofline

    common = ["--model-size", "tiny-p", "--num-requests", "5", "--max-tokens", "10", "--max-model-len", "128",
              "--max-num-seqs", "4", "--max-num-batched-tokens", "64", "--max-prefill-chunk-size", "16",
              "--block-size", "8", "--workload", "short", "--seed", "3"]
    assert benchmark.main(common + ["--temperature", "0"]) == 0
    assert "decode throughput" in capsys.readouterr().out
    assert benchmark.main(common + ["--temperature", "0.7", "--top-k", "10", "--layers", "2", "--no-pipeline"]) == 0
    capsys.readouterr()
    table = tmp_path / "roofline.json"
    assert roofline.main(["--model-size", "tiny-p", "--batch", "2", "--context", "40", "--layers", "1,3", "--steps", "4",
                          "--warmup", "1", "--block-size", "8", "--output-json", str(table)]) == 0
    rows = json.loads(table.read_text())
    assert rows[0]["us_per_layer"] > 0 and 0 < rows[0]["cache_share"] < 1 and rows[0]["size"] == "tiny-p"


def test_greedy_generation_through_the_engine(models):
    from velox_b200.engine.engine import LLM
    from velox_b200.sampling.params import SamplingParams

    folder, cfg, page, prompts, _, tensors = models["small"]
    asks = [prompts[1], prompts[2], prompts[0]]
    for dtype in ("float32", "bfloat16"):
        llm = LLM(folder, dtype=dtype, max_model_len=64, max_num_seqs=2, max_num_batched_tokens=24,
                  max_prefill_chunk_size=8, block_size=4, num_gpu_blocks=24)
        outputs = llm.generate(asks, SamplingParams(temperature=0.0, max_tokens=9, ignore_eos=True))
        for prompt, output in zip(asks, outputs):
            assert len(output) == 9
            rows = plain.forward_logits(tensors, cfg, prompt + output[:-1])[len(prompt) - 1 :]
            if dtype == "float32":
                assert output == rows.argmax(-1).tolist()
            else:
                for row, token in zip(rows, output):
                    assert row[token] >= row.max() - 3e-2 * row.abs().max()
