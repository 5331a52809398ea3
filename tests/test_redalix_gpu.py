"""The Redalix design in the engine against the plain implementation in ``plain_redalix``.

First each mechanism's kernels alone (pair rotation and cache write, the head gate, the
convolution with its state, the recurrence's gates and scan, the state-space scan, the gated
group norm, the joined norms of two results, the activations, the experts chosen by table, the
merge with a sink), then whole models through trace replay: whole prompts, the last tokens
decoded one by one, portions down to two tokens, mixed batches in a pool so small that pages and
slots are used again, long decoding, the first tokens, keys just inside and just outside a
window and the kept first keys, a sink that matters, and greedy generation through the engine's
entry point and scheduler.
"""
import numpy as np
import pytest
import torch

import plain_redalix as plain
import redalix_configs as rc
from helpers import check_logits as _check_logits, random_prompts

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def check_logits(got, want, dtype, what):
    _check_logits(got, torch.from_numpy(np.asarray(want)), dtype, what, bf16_tolerance=6e-2, bf16_min_cosine=0.997)


def close(got, want, dtype, what, scale=None):
    got = got.double().cpu()
    want = torch.as_tensor(np.asarray(want)).double()
    scale = float(want.abs().max()) if scale is None else scale
    tol = (4e-6 if dtype == "float32" else 1.2e-2) * max(scale, 1e-6)
    err = float((got - want).abs().max())
    assert err <= tol, f"{what} ({dtype}): max error {err:.3e}, allowed {tol:.3e}"


def step_arrays(lengths, slots):
    starts = np.concatenate([[0], np.cumsum(lengths)[:-1]]).astype(np.int32)
    as_dev = lambda a: torch.tensor(np.asarray(a, dtype=np.int32)).cuda()
    return as_dev(starts), as_dev(lengths), as_dev(slots)


# ------------------------------------------------------------------------------------ kernels
@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("taps,channels", [(4, 40), (1, 8), (5, 130), (2, 33)])
def test_convolution_with_state_in_portions(dtype, taps, channels):
    """A sequence's convolution cut into portions (one of a single token, one shorter than the
    taps) beside another sequence's, equals the convolution of the whole sequences."""
    from velox_b200.ops import kernels

    dt = DTYPES[dtype]
    gen = torch.Generator().manual_seed(taps * 100 + channels)
    seqs = [torch.randn(23, channels, generator=gen).to(dt), torch.randn(9, channels, generator=gen).to(dt)]
    w = torch.randn(channels, taps, generator=gen)
    b = torch.randn(channels, generator=gen)
    want = [plain.causal_conv(s.double().numpy(), w.double().numpy(), b.double().numpy()) for s in seqs]
    state = torch.randn(4, max((taps - 1) * channels, 1) + 3).cuda()
    state[1].zero_()
    state[2].zero_()
    done = [0, 0]
    got = [np.zeros((23, channels)), np.zeros((9, channels))]
    for cuts in ([5, 3], [1, 1], [2, 2], [15, 3]):
        pad = 3
        x = torch.zeros(sum(cuts), channels + pad, dtype=dt).cuda()
        row = 0
        for s, n in enumerate(cuts):
            x[row : row + n, pad:] = seqs[s][done[s] : done[s] + n].cuda()
            row += n
        out = torch.zeros(sum(cuts), channels).cuda()
        q_start, q_len, slots = step_arrays(cuts, [2, 1])
        kernels.conv_tokens(x[:, pad:], w.cuda(), b.cuda(), state[:, : max((taps - 1) * channels, 1)], out, q_start,
                            q_len, slots, 2, sum(cuts), kernels.ACT_NONE)
        row = 0
        for s, n in enumerate(cuts):
            got[s][done[s] : done[s] + n] = out[row : row + n].cpu().numpy()
            done[s] += n
            row += n
    for s in range(2):
        close(torch.from_numpy(got[s]), want[s], "float32", f"sequence {s}", scale=float(np.abs(want[s]).max()))
    assert torch.all(state[:, -3:][1:3] == 0), "the state was written beyond its columns"


@pytest.mark.parametrize("width,blocks", [(48, 3), (36, 1), (256, 4), (1280, 5)])
def test_recurrence_gates_and_scan(width, blocks):
    """Gates, decay and scan of the gated linear recurrence in two steps against the plain loop."""
    from velox_b200.ops import kernels

    gen = torch.Generator().manual_seed(width)
    part = width // blocks
    T = 37
    u = torch.randn(T, width, generator=gen)
    y = torch.randn(T, width, generator=gen)
    ra = 1.5 * torch.randn(blocks, part, part, generator=gen) / part ** 0.5
    ri = 1.5 * torch.randn(blocks, part, part, generator=gen) / part ** 0.5
    ba, bi = torch.randn(blocks, part, generator=gen), torch.randn(blocks, part, generator=gen)
    lam = 1.5 * torch.randn(width, generator=gen) - 1
    ub = u.double().reshape(T, blocks, part)
    r = plain.sigmoid(np.einsum("boi,tbi->tbo", ra.double().numpy(), ub.numpy()) + ba.double().numpy()).reshape(T, width)
    i = plain.sigmoid(np.einsum("boi,tbi->tbo", ri.double().numpy(), ub.numpy()) + bi.double().numpy()).reshape(T, width)
    a = np.exp(-8.0 * r * plain.softplus(lam.double().numpy()))
    S, want = np.zeros(width), np.zeros((T, width))
    for t in range(T):
        S = a[t] * S + np.sqrt(1 - a[t] ** 2) * i[t] * u[t].double().numpy()
        want[t] = S * plain.gelu_tanh(y[t].double().numpy())
    state = torch.zeros(3, width + 5).cuda()
    got = np.zeros((T, width))
    start = 0
    for n in (20, 1, 2, 14):
        a_buf, b_buf = torch.zeros(n, width).cuda(), torch.zeros(n, width).cuda()
        kernels.rglru_gates(u[start : start + n].cuda(), ra.transpose(1, 2).contiguous().cuda(), ba.reshape(-1).cuda(),
                            ri.transpose(1, 2).contiguous().cuda(), bi.reshape(-1).cuda(), lam.cuda(), 8.0, a_buf,
                            b_buf, n, w_a=ra.cuda(), w_i=ri.cuda())
        out = torch.zeros(n, width).cuda()
        q_start, q_len, slots = step_arrays([n], [1])
        kernels.rglru_scan(a_buf, b_buf, y[start : start + n].cuda(), state[:, 2 : 2 + width], out, q_start, q_len, slots,
                           1, kernels.ACT_GELU_TANH)
        got[start : start + n] = out.cpu().numpy()
        start += n
    close(torch.from_numpy(got), want, "float32", "recurrence", scale=float(np.abs(want).max()))
    close(state[1, 2 : 2 + width], S, "float32", "state")
    assert torch.all(state[0] == 0) and torch.all(state[2] == 0) and torch.all(state[1, :2] == 0)


@pytest.mark.parametrize("width", [40, 300])
def test_recurrence_scan_in_chunks_equals_the_loop(width):
    """Two sequences of a step, one of several chunks with a ragged end, from states that are not
    zero: the chunked form against the plain loop, outputs and final states."""
    from velox_b200.ops import kernels

    gen = torch.Generator().manual_seed(width)
    lengths = [3, 210, 64, 1]
    T = sum(lengths)
    a = torch.rand(T, width, generator=gen) * 0.6 + 0.39
    b = torch.randn(T, width, generator=gen)
    y = torch.randn(T, width, generator=gen)
    state = torch.randn(6, width + 3, generator=gen).cuda()
    before = state.clone()
    slots = [4, 0, 2, 5]
    want, row = np.zeros((T, width)), 0
    final = {}
    for n, slot in zip(lengths, slots):
        S = before[slot, 3:].double().cpu().numpy()
        for i in range(n):
            S = a[row].double().numpy() * S + b[row].double().numpy()
            want[row] = S * y[row].double().numpy()
            row += 1
        final[slot] = S
    out = torch.zeros(T, width).cuda()
    q_start, q_len, seq_slots = step_arrays(lengths, slots)
    scratch = torch.zeros(kernels.rglru_scan_scratch(T, len(lengths), width)).cuda()
    kernels.rglru_scan(a.cuda(), b.cuda(), y.cuda(), state[:, 3:], out, q_start, q_len, seq_slots, len(lengths),
                       kernels.ACT_NONE, scratch=scratch, num_tokens=T)
    close(out, want, "float32", "chunked scan", scale=float(np.abs(want).max()))
    for slot, S in final.items():
        close(state[slot, 3:], S, "float32", f"state of slot {slot}")
    assert torch.equal(state[1], before[1]) and torch.equal(state[3], before[3]) and torch.equal(state[:, :3], before[:, :3])


@pytest.mark.parametrize("heads,groups,N,P", [(4, 2, 12, 8), (3, 1, 7, 20), (8, 2, 64, 32), (2, 2, 128, 64)])
def test_state_space_scan(heads, groups, N, P):
    from velox_b200.ops import kernels

    gen = torch.Generator().manual_seed(N + P)
    T, inner = 29, heads * P
    xbc = torch.randn(T, inner + 2 * groups * N, generator=gen)
    dt_raw = torch.randn(T, heads, generator=gen)
    dt_bias, a_log, d = torch.randn(heads, generator=gen) - 1, 0.7 * torch.randn(heads, generator=gen) - 0.5, torch.randn(heads, generator=gen)
    x = xbc[:, :inner].double().numpy().reshape(T, heads, P)
    B = xbc[:, inner : inner + groups * N].double().numpy().reshape(T, groups, N)
    C = xbc[:, inner + groups * N :].double().numpy().reshape(T, groups, N)
    dt = plain.softplus(dt_raw.double().numpy() + dt_bias.double().numpy())
    want = np.zeros((T, heads, P))
    final = np.zeros((heads, N, P))
    for h in range(heads):
        g = h // (heads // groups)
        S = np.zeros((N, P))
        for t in range(T):
            S = np.exp(-np.exp(float(a_log[h])) * dt[t, h]) * S + dt[t, h] * np.outer(B[t, g], x[t, h])
            want[t, h] = S.T @ C[t, g] + float(d[h]) * x[t, h]
        final[h] = S
    state = torch.zeros(2, heads * N * P).cuda()
    got = np.zeros((T, inner))
    start = 0
    for n in (9, 1, 2, 17):
        y = torch.zeros(n, inner).cuda()
        q_start, q_len, slots = step_arrays([n], [1])
        kernels.ssd_scan(xbc[start : start + n].cuda(), dt_raw[start : start + n].cuda(), dt_bias.cuda(), a_log.cuda(),
                         d.cuda(), state, y, heads, groups, N, P, q_start, q_len, slots, 1)
        got[start : start + n] = y.cpu().numpy()
        start += n
    close(torch.from_numpy(got), want.reshape(T, inner), "float32", "state-space scan", scale=float(np.abs(want).max()))
    close(state[1], final.reshape(-1), "float32", "final state")
    assert torch.all(state[0] == 0)


def test_state_space_scan_in_chunks_equals_one_block_per_sequence():
    """Sequences of several chunks with ragged ends beside short ones, from states that are not
    zero: the three-launch form gives what the one-launch form gives."""
    from velox_b200.ops import kernels

    gen = torch.Generator().manual_seed(5)
    heads, groups, N, P = 4, 2, 24, 16
    lengths, slots = [2, 700, 256, 1, 300], [3, 0, 5, 1, 4]
    T, inner = sum(lengths), heads * P
    xbc = torch.randn(T, inner + 2 * groups * N, generator=gen).cuda()
    dt_raw = torch.randn(T, heads, generator=gen).cuda()
    dt_bias, a_log, d = (torch.randn(heads, generator=gen) - 1).cuda(), (0.7 * torch.randn(heads, generator=gen) - 2).cuda(), torch.randn(heads, generator=gen).cuda()
    state0 = torch.randn(7, heads * N * P, generator=gen).cuda()
    q_start, q_len, seq_slots = step_arrays(lengths, slots)
    results = []
    for chunked in (False, True):
        state = state0.clone()
        y = torch.zeros(T, inner).cuda()
        scratch = torch.zeros(kernels.ssd_scan_scratch(T, len(lengths), heads, N, P)).cuda() if chunked else None
        kernels.ssd_scan(xbc, dt_raw, dt_bias, a_log, d, state, y, heads, groups, N, P, q_start, q_len, seq_slots,
                         len(lengths), scratch=scratch, num_tokens=T)
        results.append((y.cpu(), state.cpu()))
    close(results[1][0], results[0][0].numpy(), "float32", "outputs", scale=float(results[0][0].abs().max()) * 4)
    close(results[1][1], results[0][1].numpy(), "float32", "states", scale=float(results[0][1].abs().max()) * 4)
    assert torch.equal(results[1][1][2], state0[2].cpu()) and torch.equal(results[1][1][6], state0[6].cpu())


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_row_kernels(dtype):
    """Gated group norm, the mean of two normed results, activations, the gate on rows."""
    from velox_b200.ops import kernels

    dt = DTYPES[dtype]
    gen = torch.Generator().manual_seed(4)
    T, inner, parts = 6, 120, 3
    y = torch.randn(T, inner, generator=gen).cuda()
    z = torch.randn(T, inner + 8, generator=gen).to(dt).cuda()
    w = (1 + 0.2 * torch.randn(inner, generator=gen)).cuda()
    out = torch.zeros(T, inner, dtype=dt).cuda()
    kernels.gated_group_norm(y, z[:, 8:], w, 1e-5, parts, out, T)
    v = y.double().cpu().numpy() * plain.silu(z[:, 8:].double().cpu().numpy())
    want = plain.rms_norm(v.reshape(T, parts, inner // parts), None, 1e-5).reshape(T, inner) * w.double().cpu().numpy()
    close(out, want, dtype, "gated group norm")

    a = (3 * torch.randn(T, 100, generator=gen)).to(dt).cuda()
    b = (0.1 * torch.randn(T, 100, generator=gen)).to(dt).cuda()
    wa, wb = (1 + 0.2 * torch.randn(100, generator=gen)).cuda(), (1 + 0.2 * torch.randn(100, generator=gen)).cuda()
    resid = torch.randn(T, 100, generator=gen).cuda()
    before = resid.double().cpu().numpy()
    mean = 0.5 * (plain.rms_norm(a.double().cpu().numpy(), wa.double().cpu().numpy(), 1e-6)
                  + plain.rms_norm(b.double().cpu().numpy(), wb.double().cpu().numpy(), 1e-6))
    kernels.dual_norm_mean(a, b, wa, wb, 1e-6, 0.5, T, resid=resid)
    close(resid, before + mean, "float32" if dtype == "float32" else dtype, "mean of two normed results into the stream")
    other = torch.zeros(T, 100, dtype=dt).cuda()
    kernels.dual_norm_mean(a, b, wa, wb, 1e-6, 0.5, T, out=other)
    close(other, mean, dtype, "mean of two normed results")

    wide = torch.linspace(-6, 6, 77).repeat(T, 1).to(dt).cuda()
    for kind, fn in ((kernels.ACT_GELU_TANH, plain.gelu_tanh), (kernels.ACT_RELU_SQUARED, plain.relu_squared),
                     (kernels.ACT_SILU, plain.silu)):
        act = torch.zeros(T, 80, dtype=dt).cuda()
        kernels.act_rows(wide[:, 5:], act[:, :72], T, kind)
        close(act[:, :72], fn(wide[:, 5:].double().cpu().numpy()), dtype, f"activation {kind}", scale=36.0 if kind == 3 else 6.0)
        assert torch.all(act[:, 72:] == 0)

    logits = torch.randn(T, 9, generator=gen).to(dt).cuda()
    x = torch.randn(T, 100, generator=gen).to(dt).cuda()
    resid = torch.randn(T, 100, generator=gen).cuda()
    want = resid.double().cpu().numpy() + plain.sigmoid(logits[:, 4:5].double().cpu().numpy()) * x.double().cpu().numpy()
    kernels.gated_rows_add(resid, x, logits[:, 4:5], T)
    close(resid, want, "float32", "gated rows into the stream", scale=1e3 if dtype == "bfloat16" else None)


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("width,ff,experts,top", [(64, 24, 5, 2), (100, 17, 3, 1), (256, 64, 8, 3)])
def test_experts_by_table(dtype, width, ff, experts, top):
    from velox_b200.ops import kernels

    dt = DTYPES[dtype]
    gen = torch.Generator().manual_seed(width + ff)
    vocab, T = 50, 11
    h = torch.randn(T, width + 8, generator=gen).to(dt).cuda()
    up = (torch.randn(experts, ff, width, generator=gen) / width ** 0.5).to(dt).cuda()
    down = (torch.randn(experts, width, ff, generator=gen) / ff ** 0.5).to(dt).cuda()
    table = torch.rand(vocab, experts, generator=gen).argsort(dim=1)[:, :top].to(torch.int32).contiguous().cuda()
    ids = torch.randint(0, vocab, (T,), generator=gen).to(torch.int32)
    fed = torch.tensor([7, 3], dtype=torch.int32).cuda()
    ids[4] = -2  # stands for fed[1]
    resid = torch.randn(T, width, generator=gen).cuda()
    want = resid.double().cpu().numpy()
    hs = h[:, 8:].double().cpu().numpy()
    for t in range(T):
        token = int(ids[t]) if ids[t] >= 0 else int(fed[-1 - int(ids[t])])
        for e in table[token].tolist():
            want[t] += plain.relu_squared(hs[t] @ up[e].double().cpu().numpy().T) @ down[e].double().cpu().numpy().T / top
    status = torch.zeros(4, dtype=torch.int32).cuda()
    start = resid.clone()
    loose = float(np.abs(want).max()) * (1 if dtype == "float32" else 30)
    kernels.table_experts(h[:, 8:], ids.cuda(), fed, table, up, down, resid, T, status)
    assert int(status[0]) == 0
    close(resid, want, "float32", "experts by table", scale=loose)
    # the same as matrix-vector products spread over the grid
    resid2 = start.clone()
    act = torch.zeros(T * top * ff).cuda()
    assert kernels.table_experts_rows(h[:, 8:], ids.cuda(), fed, table, up, down, act, resid2, T, status)
    close(resid2, want, "float32", "experts by table, rows over the grid", scale=loose)
    # and as tiled products over the pairs ordered by expert (activations rounded to bfloat16)
    if dtype == "bfloat16" and width % 8 == 0 and ff % 8 == 0:
        places = kernels.grouped_places(T, top, experts)
        route = torch.zeros(2 * places + T * top, dtype=torch.int32).cuda()
        acts = torch.zeros(places, ff, dtype=torch.bfloat16).cuda()
        rows = torch.zeros(places, width).cuda()
        resid3 = start.clone()
        assert kernels.table_experts_grouped(h[:, 8:], ids.cuda(), fed, table, up, down, route, acts, rows, resid3, T, status)
        close(resid3, want, "float32", "experts by table, grouped", scale=float(np.abs(want).max()) * 3000)
    assert int(status[0]) == 0


@pytest.mark.parametrize("tokens,width,ff,experts,top", [(300, 64, 24, 5, 2), (130, 256, 72, 8, 3), (700, 128, 200, 16, 1)])
def test_experts_grouped_many_tokens(tokens, width, ff, experts, top):
    """Runs of many tokens per expert (several tiles, ragged ends, an expert nobody names)."""
    from velox_b200.ops import kernels

    gen = torch.Generator().manual_seed(tokens)
    vocab = 40
    h = torch.randn(tokens, width, generator=gen).to(torch.bfloat16).cuda()
    up = (torch.randn(experts, ff, width, generator=gen) / width ** 0.5).to(torch.bfloat16).cuda()
    down = (torch.randn(experts, width, ff, generator=gen) / ff ** 0.5).to(torch.bfloat16).cuda()
    table = torch.rand(vocab, experts - 1, generator=gen).argsort(dim=1)[:, :top].to(torch.int32).contiguous().cuda()
    ids = torch.randint(0, vocab, (tokens,), generator=gen).to(torch.int32).cuda()
    resid = torch.randn(tokens, width, generator=gen).cuda()
    want = resid.double()
    chosen = table[ids.long()].long()
    for k in range(top):
        a = torch.relu(torch.einsum("tw,tfw->tf", h.double(), up.double()[chosen[:, k]])) ** 2
        want = want + torch.einsum("tf,twf->tw", a.to(torch.bfloat16).double(), down.double()[chosen[:, k]]) / top
    places = kernels.grouped_places(tokens, top, experts)
    route = torch.zeros(2 * places + tokens * top, dtype=torch.int32).cuda()
    acts = torch.zeros(places, ff, dtype=torch.bfloat16).cuda()
    rows = torch.zeros(places, width).cuda()
    status = torch.zeros(4, dtype=torch.int32).cuda()
    assert kernels.table_experts_grouped(h, ids, None, table, up, down, route, acts, rows, resid, tokens, status)
    assert int(status[0]) == 0
    close(resid, want.cpu().numpy(), "float32", "grouped experts", scale=float(want.abs().max()) * 300)


@pytest.mark.parametrize("tokens,width,ff,experts,top", [(500, 128, 96, 6, 2), (300, 256, 64, 9, 3), (1100, 64, 32, 4, 1)])
def test_experts_with_the_library_grouped_product(tokens, width, ff, experts, top):
    """The long-step form whose two products are the library's grouped product, around this
    package's ordering, gather, activation and sum; an expert nobody names has an empty run."""
    from velox_b200.ops import kernels

    if not kernels.has_library_grouped_product():
        pytest.skip("this torch has no grouped product")
    gen = torch.Generator().manual_seed(tokens + 1)
    vocab = 40
    h = torch.randn(tokens, width + 8, generator=gen).to(torch.bfloat16).cuda()
    up = (torch.randn(experts, ff, width, generator=gen) / width ** 0.5).to(torch.bfloat16).cuda()
    down = (torch.randn(experts, width, ff, generator=gen) / ff ** 0.5).to(torch.bfloat16).cuda()
    table = (1 + torch.rand(vocab, experts - 1, generator=gen).argsort(dim=1)[:, :top]).to(torch.int32).contiguous().cuda()
    ids = torch.randint(0, vocab, (tokens,), generator=gen).to(torch.int32).cuda()
    resid = torch.randn(tokens, width, generator=gen).cuda()
    want = resid.double()
    chosen = table[ids.long()].long()
    x = h[:, 8:]
    for k in range(top):
        a = torch.relu(torch.einsum("tw,tfw->tf", x.double(), up.double()[chosen[:, k]]).to(torch.bfloat16).double()) ** 2
        want = want + torch.einsum("tf,twf->tw", a.to(torch.bfloat16).double(), down.double()[chosen[:, k]]) / top
    places = kernels.grouped_places(tokens, top, experts)
    route = torch.zeros(2 * places + tokens * top, dtype=torch.int32).cuda()
    ends = torch.zeros(experts, dtype=torch.int32).cuda()
    a_rows = torch.zeros(places, width, dtype=torch.bfloat16).cuda()
    status = torch.zeros(4, dtype=torch.int32).cuda()
    assert kernels.table_experts_library(x, ids, None, table, up, down, route, ends, a_rows, resid, tokens, status)
    assert int(status[0]) == 0
    assert int(ends[0]) == 0 and int(ends[-1]) <= places
    close(resid, want.cpu().numpy(), "float32", "experts through the library's grouped product",
          scale=float(want.abs().max()) * 3000)


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_pair_rotation_cache_write_and_head_gate(dtype):
    from velox_b200.ops import kernels

    dt = DTYPES[dtype]
    gen = torch.Generator().manual_seed(8)
    T, H, G, D, rot = 7, 4, 2, 32, 12
    extra = H + 4
    qkv = torch.randn(T, (H + 2 * G) * D + extra, generator=gen).to(dt).cuda()
    keep = qkv.clone()
    positions = torch.tensor([0, 5, 6, 40, 41, 3, 99], dtype=torch.int32).cuda()
    rot_cfg = {"base": 100.0, "dims": rot, "scaling": {"factor": 4.0, "original": 16, "fast": 8.0, "slow": 1.0}}
    freq, mag = plain.yarn_frequencies(rot, 100.0, rot_cfg["scaling"])
    angles = np.arange(128)[:, None] * freq[None, :]
    cos = torch.tensor(np.cos(angles) * mag, dtype=torch.float32).cuda()
    sin = torch.tensor(np.sin(angles) * mag, dtype=torch.float32).cuda()
    slots = torch.tensor([3, 9, -1, 0, 17, 20, 8], dtype=torch.int32).cuda()
    k_cache = torch.zeros(3, 8, G, D, dtype=dt).cuda()
    v_cache = torch.zeros(3, 8, G, D, dtype=dt).cuda()
    status = torch.zeros(4, dtype=torch.int32).cuda()
    kernels.pair_rope_cache_write(qkv, positions, cos, sin, slots, k_cache, v_cache, T, H, G, D, rot, status)
    assert int(status[0]) == 0
    pos = positions.cpu().numpy()
    q = plain.rotate_pairs(keep[:, : H * D].double().cpu().numpy().reshape(T, H, D), pos, rot_cfg)
    k = plain.rotate_pairs(keep[:, H * D : (H + G) * D].double().cpu().numpy().reshape(T, G, D), pos, rot_cfg)
    close(qkv[:, : H * D], q.reshape(T, -1), dtype, "rotated queries")
    assert torch.equal(qkv[:, H * D :], keep[:, H * D :]), "columns behind the queries changed"
    flat_k, flat_v = k_cache.view(-1, G, D), v_cache.view(-1, G, D)
    for t in range(T):
        s = int(slots[t])
        if s < 0:
            continue
        close(flat_k[s], k[t], dtype, f"key of token {t}")
        assert torch.equal(flat_v[s].reshape(-1), keep[t, (H + G) * D : (H + 2 * G) * D])
    assert torch.all(flat_k[1] == 0)
    out = torch.randn(T, H * D, generator=gen).to(dt).cuda()
    want = out.double().cpu().numpy().reshape(T, H, D) * plain.sigmoid(
        keep[:, (H + 2 * G) * D : (H + 2 * G) * D + H].double().cpu().numpy())[:, :, None]
    kernels.head_gate(out, qkv[:, (H + 2 * G) * D : (H + 2 * G) * D + H], T, H, D)
    close(out, want.reshape(T, -1), dtype, "gated heads")


# ------------------------------------------------------------------------------------ models
CASES = {
    "small": (rc.SMALL, 4, (5, 11, 17, 60, 100), 2.0),
    "odd": (rc.ODD, 16, (1, 9, 33, 70, 150), 1.5),
    "wide": (rc.WIDE, 64, (130, 3, 65, 300, 64), 2.5),
}


def reference(cfg, tensors, tokens, collect=None):
    return plain.forward(cfg, rc.as_numpy(tensors), tokens, collect)


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, (cfg, page, lengths, sharp) in CASES.items():
        folder = str(tmp_path_factory.mktemp("redalix_" + name))
        tensors = rc.make_weights(cfg, seed=5 + len(name), sharp=sharp)
        rc.write_folder(folder, cfg, tensors)
        prompts = random_prompts(cfg["vocab"], lengths, seed=31)
        want = [reference(cfg, tensors, p) for p in prompts]
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
        if L > 2:
            portions = replay_one(replayer, f"p{index}", tokens, changing_cuts(L))
            check_logits(portions, ref, dtype, f"{case} request {index} in portions")
    replayer.cache.assert_consistent()
    assert replayer.cache.num_free_pages() == replayer.cache.num_total_pages
    assert replayer.cache.num_free_slots == replayer.max_live


def test_layer_streams(models):
    """The stream after every layer of the float32 path against the plain implementation's."""
    folder, cfg, page, prompts, _, tensors = models["odd"]
    tokens = prompts[3]
    streams = []
    reference(cfg, tensors, tokens, streams)
    replayer = make_replayer(folder, "float32", max_tokens=128, page=page, enable_graphs=False)
    seen = []
    for block in replayer.model.blocks:
        def wrapped(hidden, ctx, cache, inner=block.forward):
            inner(hidden, ctx, cache)
            x = hidden.resid[: ctx.num_tokens].clone()
            if hidden.delta is not None:
                x += hidden.delta[: ctx.num_tokens].float()
            seen.append(x.double().cpu())
        block.forward = wrapped
    replay_one(replayer, "s", tokens, [len(tokens)])
    assert len(seen) == len(streams)
    for index, (got, want) in enumerate(zip(seen, streams)):
        close(got, want, "float32", f"stream after layer {index}", scale=8 * float(np.abs(want).max()))


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
    """Every request twice, up to four live at a time in a pool that holds no more: a request's
    logits equal those of the request alone whatever shares its steps, and a slot's state and a
    page's keys of an earlier request do not leak into a later one."""
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
    assert replayer.cache.num_free_pages() == replayer.cache.num_total_pages
    assert set(slots_used) <= set(range(4))


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("case,page", [("small", 4), ("wide", 16)])
def test_long_decode(models, case, page, dtype):
    folder, cfg, _, _, _, tensors = models[case]
    tokens = random_prompts(cfg["vocab"], [420], seed=4)[0]
    ref = reference(cfg, tensors, tokens)
    replayer = make_replayer(folder, dtype, max_tokens=448, page=page)
    rows = replay_one(replayer, "long", tokens, [30] + [1] * 390)
    check_logits(rows, ref, dtype, "long decode")
    # the windows have passed pages that were given back; the kept first keys' pages were not
    replayer.cache.assert_consistent()


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_long_prompt_whole_and_in_large_portions(models, dtype):
    folder, cfg, page, _, _, tensors = models["wide"]
    tokens = random_prompts(cfg["vocab"], [600], seed=14)[0]
    ref = reference(cfg, tensors, tokens)
    replayer = make_replayer(folder, dtype, max_tokens=640, page=page)
    check_logits(replay_one(replayer, "whole", tokens, [600]), ref, dtype, "600 tokens whole")
    check_logits(replay_one(replayer, "parts", tokens, [300, 299, 1]), ref, dtype, "600 tokens as 300 + 299 + 1")


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_first_tokens(models, dtype):
    folder, cfg, page, prompts, want, _ = models["odd"]
    replayer = make_replayer(folder, dtype, max_tokens=64, page=page)
    rows = replay_one(replayer, "f", prompts[3][:6], [1, 1, 2, 2])
    check_logits(rows, want[3][:6], dtype, "first tokens")


def needle_model(tmp_path, kind):
    """A one-layer model whose attention puts nearly all weight of an ``asker`` token's query on a
    ``marker`` token's key, wherever it is: q and k of the first head pair line up with the two
    tokens' normed embeddings.  ``kind`` parallel: window 40 with 6 kept first keys and a sink;
    attention: window 40, rotation of 4 of 16 dims only, so that the needle's score does not
    depend on the distance."""
    width, vocab = 64, 90
    if kind == "parallel":
        layer = rc.parallel(rc.attention(2, 1, 16, 16, 1.0, 40, keep_first=6), rc.recurrence(32, 2, 2), None)
        prefix = "l0.mix.left."
    else:
        layer = rc.attn_layer(rc.attention(2, 1, 16, 16, 1.0, 40, rot=rc.rotation(100.0, 4)), None)
        prefix = "l0.mix."
    cfg = rc.config(width, vocab, [layer])
    tensors = {k: (v if v.dtype == torch.int32 else v.float()) for k, v in rc.make_weights(cfg, seed=2).items()}
    marker, asker = 7, 11
    tensors["l0.norm1"] = torch.ones(width)
    unit = lambda v: v / (v.pow(2).mean().sqrt())  # what the RMS norm makes of an embedding row
    q = tensors[prefix + "q"].view(2, 16, width)
    k = tensors[prefix + "k"].view(1, 16, width)
    q[:, 8] = 0.35 * unit(tensors["embed"][asker]) / width ** 0.5 * 8
    k[:, 8] = 0.35 * unit(tensors["embed"][marker]) / width ** 0.5 * 8
    if prefix + "q.b" in tensors:
        tensors[prefix + "q.b"].zero_()
        tensors[prefix + "k.b"].zero_()
    tensors = {k_: (v if v.dtype == torch.int32 else v.to(torch.bfloat16)) for k_, v in tensors.items()}
    folder = str(tmp_path / f"needle_{kind}")
    rc.write_folder(folder, cfg, tensors)
    return folder, cfg, tensors, marker, asker


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("kind,needle_at,seen", [
    ("parallel", 0, True), ("parallel", 5, True), ("parallel", 6, False), ("parallel", 63, False),
    ("parallel", 279, False), ("parallel", 280, True), ("parallel", 300, True),
    ("attention", 0, False), ("attention", 279, False), ("attention", 280, True), ("attention", 255, False),
    ("attention", 256, False), ("attention", 318, True),
])
def test_keys_at_the_edges_of_window_and_kept_first(tmp_path, dtype, kind, needle_at, seen):
    """A key that takes nearly all softmax weight of the query at position 319 when it is seen:
    just inside and just outside the window of 40 (positions 280 and 279), among the kept first
    keys and just behind them (5 and 6), at page borders; decoded and inside a portion."""
    folder, cfg, tensors, marker, asker = needle_model(tmp_path, kind)
    length = 330
    tokens = [t if t not in (marker, asker) else 20 for t in random_prompts(90, [length], seed=needle_at)[0]]
    tokens[needle_at] = marker
    tokens[319] = asker
    ref = reference(cfg, tensors, tokens)
    without = list(tokens)
    without[needle_at] = 21
    other = reference(cfg, tensors, without)
    moved = float(np.abs(other[319] - ref[319]).max())
    if seen:
        assert moved > 0.3, f"the needle does not matter enough for this test ({moved:.3f})"
    else:
        assert moved < 0.05 or kind == "parallel", f"a key outside the window matters ({moved:.3f})"
    replayer = make_replayer(folder, dtype, max_tokens=384, page=64)
    rows = replay_one(replayer, "n", tokens, [319, 1, 10])
    check_logits(rows[316:323], ref[316:323], dtype, f"{kind} needle at {needle_at}, decoded")
    rows = replay_one(replayer, "m", tokens, [100, 2, 200, 28])
    check_logits(rows[316:323], ref[316:323], dtype, f"{kind} needle at {needle_at}, in portions")
    rows = replay_one(replayer, "w", tokens, [length])
    check_logits(rows[316:323], ref[316:323], dtype, f"{kind} needle at {needle_at}, whole")


def test_the_sink_matters(tmp_path):
    """With large sinks the attention's output shrinks; the engine follows the plain model for
    sinks of -30 (no effect), 0 and +6 (most of the weight)."""
    cfg = rc.config(64, 80, [rc.parallel(rc.attention(4, 2, 16, 16, 0.25, 20, keep_first=2), rc.recurrence(32, 2, 3),
                                         rc.dense(32))])
    base = rc.make_weights(cfg, seed=3, sharp=2.0)
    tokens = random_prompts(80, [70], seed=6)[0]
    rows = []
    for value in (-30.0, 0.0, 6.0):
        tensors = dict(base)
        tensors["l0.mix.left.sink"] = torch.full((4,), value).to(torch.bfloat16)
        folder = str(tmp_path / f"sink{int(value)}")
        rc.write_folder(folder, cfg, tensors)
        ref = reference(cfg, tensors, tokens)
        rows.append(ref)
        for dtype in DTYPES:
            replayer = make_replayer(folder, dtype, max_tokens=128, page=16)
            check_logits(replay_one(replayer, "a", tokens, [40, 1, 1, 28]), ref, dtype, f"sink {value}")
    assert np.abs(rows[0] - rows[2]).max() > 0.2, "the sink does not matter enough for this test"


def test_command_lines_take_the_design(tmp_path, capsys):
    import json

    from velox_b200.cli import benchmark, roofline

    common = ["--model-size", "tiny-r", "--num-requests", "5", "--max-tokens", "10", "--max-model-len", "128",
              "--max-num-seqs", "4", "--max-num-batched-tokens", "64", "--max-prefill-chunk-size", "16",
              "--block-size", "8", "--workload", "short", "--seed", "3"]
    assert benchmark.main(common + ["--temperature", "0"]) == 0
    assert "decode throughput" in capsys.readouterr().out
    assert benchmark.main(common + ["--temperature", "0.7", "--top-k", "10", "--no-pipeline"]) == 0
    capsys.readouterr()
    table = tmp_path / "roofline.json"
    assert roofline.main(["--model-size", "tiny-r", "--batch", "2", "--context", "40", "--layers", "3,6", "--steps", "4",
                          "--warmup", "1", "--block-size", "8", "--output-json", str(table)]) == 0
    rows = json.loads(table.read_text())
    assert rows[0]["us_per_layer"] > 0 and rows[0]["size"] == "tiny-r"


def test_greedy_generation_through_the_engine(models):
    from velox_b200.engine.engine import LLM
    from velox_b200.sampling.params import SamplingParams

    folder, cfg, page, prompts, _, tensors = models["small"]
    asks = [prompts[1], prompts[2], prompts[0], prompts[3]]
    for dtype in ("float32", "bfloat16"):
        llm = LLM(folder, dtype=dtype, max_model_len=96, max_num_seqs=2, max_num_batched_tokens=24,
                  max_prefill_chunk_size=8, block_size=4, num_gpu_blocks=40)
        outputs = llm.generate(asks, SamplingParams(temperature=0.0, max_tokens=9, ignore_eos=True))
        for prompt, output in zip(asks, outputs):
            assert len(output) == 9
            rows = reference(cfg, tensors, prompt + output[:-1])[len(prompt) - 1 :]
            if dtype == "float32":
                assert output == rows.argmax(-1).tolist()
            else:
                for row, token in zip(rows, output):
                    assert row[token] >= row.max() - 3e-2 * np.abs(row).max()
