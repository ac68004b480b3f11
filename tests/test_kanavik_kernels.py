"""The score-mixing attention kernels and the gated scan alone, each against its plain PyTorch
statement, at sizes other than any model's: both attention kernels (a CTA per token; the tiled one
with and without its keys split), steps of prompt portions beside single tokens, windows whose edge
falls inside a tile, and the scan in one piece and in segments."""
import pytest
import torch

import kernel_references as ref
from test_gpu_kernels import _attention_case, status, tol

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    return torch.device("cuda:0")


def _step_split(requests):
    """q_tiles and the indices of single tokens for requests given as (start, q_len)."""
    tiles, singles, token = [], [], 0
    for r, (start, q_len) in enumerate(requests):
        if q_len == 1:
            singles.append(token)
        else:
            for first in range(0, q_len, 128):
                tiles.append((r, token + first, min(128, q_len - first), start + first))
        token += q_len
    return (torch.tensor(tiles, dtype=torch.int32).view(-1, 4), torch.tensor(singles, dtype=torch.int32))


def _mixing(heads, generator, dev):
    slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)])
    talk = torch.eye(heads) + 0.3 * torch.randn((heads, heads), generator=generator)
    sink = torch.randn((heads,), generator=generator)
    return slopes.to(dev), talk.to(dev), sink.to(dev)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads, kv_heads, size, vsize, page_size", [
    (4, 2, 16, 16, 4), (3, 1, 32, 24, 8), (14, 2, 64, 64, 16), (6, 3, 48, 40, 16), (8, 8, 128, 128, 16),
    (5, 5, 20, 100, 3), (1, 1, 64, 8, 64), (17, 1, 8, 36, 16), (32, 4, 64, 64, 16),
])
@pytest.mark.parametrize("window", [None, 5, 70])
@pytest.mark.parametrize("parts", ["all", "no sink", "plain"])
def test_tiled_score_mixing_attention(dev, dtype, heads, kv_heads, size, vsize, page_size, window, parts):
    from einf_b200 import ops

    if parts != "all" and (window != 70 or dtype != torch.float32):
        pytest.skip("the optional parts are switched off in one setting")
    requests = [(0, 1), (0, 2 * page_size), (3, 6), (15, 2), (page_size * 4 - 1, 1), (200, 1), (0, 137), (61, 19),
                (130, 70)]
    (q, k, v, table, seq, pos), scale, window = _attention_case(dev, dtype, heads, kv_heads, size, page_size, requests, window)
    generator = torch.Generator().manual_seed(5)
    v = torch.randn((*v.shape[:3], vsize), generator=generator).to(dtype).to(dev)
    slopes, talk, sink = _mixing(heads, generator, dev)
    if parts == "no sink":
        sink = None
    if parts == "plain":
        slopes = talk = sink = None
    q_tiles, singles = _step_split(requests)
    want = torch.empty((q.shape[0], heads, vsize), dtype=dtype, device=dev)
    st = status(dev)
    ref.paged_attention_mixed(q.cpu(), k.cpu(), v.cpu(), table.cpu(), seq.cpu(), pos.cpu(), want_cpu := want.cpu(), scale,
                              window, *(None if t is None else t.cpu() for t in (slopes, talk, sink)), 0.7, st.cpu())
    close = dict(rtol=2e-4, atol=2e-5) if dtype == torch.float32 else tol(dtype)
    for tiled in (False, True):
        out = torch.full_like(want, float("nan"))
        extra = dict(q_tiles=q_tiles.to(dev), single_tokens=singles.to(dev), num_singles=singles.shape[0],
                     max_context=max(s + n for s, n in requests)) if tiled else {}
        if tiled:
            assert ops.mixed_tiled_rows(heads, kv_heads, size, vsize, False) and ops.mixed_tiled_rows(heads, kv_heads, size, vsize, True)
        ops.paged_attention_mixed(q, k, v, table, seq, pos, out, scale, window, slopes, talk, sink, 0.7, st, **extra)
        assert int(st) == 0
        torch.testing.assert_close(out.cpu(), want_cpu, **close)


@pytest.mark.parametrize("batch, context, window", [(1, 3000, None), (3, 1500, 1024), (64, 300, 128), (2, 40, 64)])
def test_tiled_score_mixing_decode_splits_its_keys(dev, batch, context, window):
    """Single tokens with long contexts: the keys of a token are split over CTAs and joined with the sink."""
    from einf_b200 import ops

    heads, kv_heads, size, page_size = 6, 2, 32, 16
    requests = [(context - 1 - 7 * (r % 5), 1) for r in range(batch)]
    (q, k, v, table, seq, pos), scale, window = _attention_case(dev, torch.bfloat16, heads, kv_heads, size, page_size,
                                                                requests, window)
    generator = torch.Generator().manual_seed(9)
    slopes, talk, sink = _mixing(heads, generator, dev)
    assert ops.mixed_tiled_splits(batch, 1, window, context) > 1 or context < 128
    out, want = torch.empty_like(q), torch.empty_like(q).cpu()
    st = status(dev)
    ops.paged_attention_mixed(q, k, v, table, seq, pos, out, scale, window, slopes, talk, sink, 1.0, st,
                              q_tiles=torch.zeros((0, 4), dtype=torch.int32, device=dev), single_tokens=None,
                              num_singles=batch, max_context=context)
    ref.paged_attention_mixed(q.cpu(), k.cpu(), v.cpu(), table.cpu(), seq.cpu(), pos.cpu(), want, scale, window,
                              slopes.cpu(), talk.cpu(), sink.cpu(), 1.0, st.cpu())
    assert int(st) == 0
    torch.testing.assert_close(out.cpu(), want, **tol(torch.bfloat16))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_tiled_score_mixing_far_key_and_window_edge(dev, dtype):
    """One key far back carries the weight: a query whose window still holds it returns its value, the next
    query, for which it has just left the window, does not; in a prompt portion and for a single token."""
    from einf_b200 import ops

    heads, kv_heads, size, page_size, window = 4, 2, 32, 16, 100
    needle = 37
    for requests in ([(0, 300)], [(needle + window - 1, 1), (needle + window, 1)], [(100, 60)]):
        (q, k, v, table, seq, pos), scale, _ = _attention_case(dev, dtype, heads, kv_heads, size, page_size,
                                                               requests, window)
        q[:] = 0.0
        q[:, :, 0] = 1.0
        k[:] = 0.0
        for r in range(len(requests)):
            page, offset = int(table[r, needle // page_size]), needle % page_size
            k[page, :, offset, 0] = 40.0 / scale
            v[page, :, offset, :] = 7.0
        out = torch.empty_like(q)
        st = status(dev)
        q_tiles, singles = _step_split(requests)
        ops.paged_attention_mixed(q, k, v, table, seq, pos, out, scale, window, None, None, None, 1.0, st,
                                  q_tiles=q_tiles.to(dev), single_tokens=singles.to(dev), num_singles=singles.shape[0],
                                  max_context=max(s + n for s, n in requests))
        assert int(st) == 0
        for t in range(q.shape[0]):
            p = int(pos[t])
            inside = needle <= p < needle + window
            got = out[t].abs().max().item()
            assert (abs(got - 7.0) < 1e-3) if inside else got < 6.0, (dtype, requests, p, got)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("lengths", [(1, 1, 1), (5, 1, 33), (700,), (16, 17, 130, 2), (2100, 3)])
def test_gated_scan_in_segments(dev, dtype, lengths):
    from einf_b200 import ops

    blocks, part = 3, 20
    width = blocks * part
    tokens = sum(lengths)
    generator = torch.Generator().manual_seed(len(lengths) + tokens)
    gates = torch.randn((tokens, blocks, 2 * part), generator=generator)
    gate_bias = torch.randn((blocks, 2 * part), generator=generator)
    u = torch.randn((tokens, width), generator=generator).to(dtype)
    y_raw = torch.randn((tokens, width), generator=generator).to(dtype)
    y_bias = torch.randn((width,), generator=generator)
    rate = -8.0 * torch.nn.functional.softplus(torch.randn((width,), generator=generator) - 3.0)
    state = torch.randn((len(lengths) + 2, width), generator=generator)
    starts = [0]
    for n in lengths:
        starts.append(starts[-1] + n)
    q_start = torch.tensor(starts, dtype=torch.int32)
    slots = torch.tensor([(r + 1) % (len(lengths) + 2) for r in range(len(lengths))], dtype=torch.int32)
    want, want_state = torch.empty((tokens, width), dtype=dtype), state.clone()
    ref.gated_scan(gates, gate_bias, u, y_raw, y_bias, rate, want_state, q_start, slots, want, 1.3)
    got, got_state = torch.empty((tokens, width), dtype=dtype, device=dev), state.clone().to(dev)
    ops.gated_scan(gates.to(dev), gate_bias.to(dev), u.to(dev), y_raw.to(dev), y_bias.to(dev), rate.to(dev), got_state,
                   q_start.to(dev), slots.to(dev), got, 1.3, max_q_len=max(lengths))
    close = dict(rtol=2e-4, atol=2e-5) if dtype == torch.float32 else tol(dtype)
    torch.testing.assert_close(got.cpu(), want, **close)
    torch.testing.assert_close(got_state.cpu(), want_state, rtol=2e-4, atol=2e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens, hidden, side, layers_done", [
    (1, 64, 8, 0), (5, 72, 6, 2), (9, 100, 16, 1), (1030, 128, 64, 3), (8, 896, 64, 7), (3, 1544, 33, 0),
])
@pytest.mark.parametrize("parts", ["both", "token input", "depth average", "neither"])
def test_end_of_a_layer(dev, dtype, tokens, hidden, side, layers_done, parts):
    """The kernel that takes several tokens a CTA (widths that are multiples of eight) and the one that
    takes a row a CTA (the others): pending sublayer output, token input, depth average."""
    from einf_b200 import ops

    if parts != "both" and tokens not in (5, 1030):
        pytest.skip("the parts alone at two sizes")
    generator = torch.Generator().manual_seed(tokens + hidden)
    vocab = 50
    residual = torch.randn((tokens, hidden), generator=generator)
    pending = [torch.randn((tokens, hidden), generator=generator).to(dtype)]
    ids = torch.randint(0, vocab, (tokens,), generator=generator, dtype=torch.int32)
    table = torch.randn((vocab, side), generator=generator).to(dtype)
    gate = (torch.randn((side, hidden), generator=generator) * hidden ** -0.5).to(dtype)
    proj_t = torch.randn((side, hidden), generator=generator).to(dtype)
    norm = torch.rand((hidden,), generator=generator) + 0.5
    history = torch.randn((layers_done + 2, tokens, hidden), generator=generator)
    weight = torch.randn((layers_done + 2,), generator=generator)
    use_side, use_depth = parts in ("both", "token input"), parts in ("both", "depth average")

    def arguments(move):
        return (move(residual.clone()), [move(t) for t in pending], 0.6, move(ids),
                (move(table), move(gate), move(proj_t), move(norm), 1e-5) if use_side else None,
                (move(history.clone()), layers_done, move(weight)) if use_depth else None)

    want, got = arguments(lambda t: t), arguments(lambda t: t.to(dev))
    ref.stream_tail(*want)
    ops.stream_tail(*got)
    close = dict(rtol=2e-4, atol=2e-4) if dtype == torch.float32 else dict(rtol=1e-3, atol=1e-3)
    torch.testing.assert_close(got[0].cpu(), want[0], **close)
    if use_depth:
        torch.testing.assert_close(got[5][0].cpu(), want[5][0], **close)
