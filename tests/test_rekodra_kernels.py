"""The kernels that came with the Rekodra decoder, each alone against its plain PyTorch statement, at
sizes other than any model's: the store kernel's weighted norms (head by head and over whole rows)
and values taken from the keys, a sink in the general and the tensor-core attention kernels, the
router with a correction and groups, the combine with pass-through experts and a gated addend,
the matrix memory's gates and output with the recurrence between them, the normed join of
branches, the scaled embedding and the scaled logits."""
import pytest
import torch

import kernel_references as ref
from test_gpu_kernels import _attention_case, status, tol

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]


@pytest.fixture(scope="module")
def dev():
    return torch.device("cuda:0")


def test_embedding_and_logits_take_a_factor(dev):
    from einf_b200 import ops

    table = torch.randn(53, 40, device=dev).to(torch.bfloat16)
    tokens = torch.tensor([0, 52, 7, 7, 31], dtype=torch.int32, device=dev)
    out = torch.empty((5, 40), dtype=torch.float32, device=dev)
    st = status(dev)
    ops.embed(tokens, table, out, st, scale=0.37)
    torch.testing.assert_close(out, table[tokens.long()].float() * 0.37, rtol=1e-6, atol=1e-7)
    logits = torch.randn((7, 61), device=dev)
    want = logits * 0.25
    ops.softcap(logits, None, 0.25)
    torch.testing.assert_close(logits, want, rtol=1e-6, atol=1e-7)
    logits = torch.randn((7, 61), device=dev) * 20
    want = 30.0 * torch.tanh(logits * 0.5 / 30.0)
    ops.softcap(logits, 30.0, 0.5)
    torch.testing.assert_close(logits, want, rtol=1e-5, atol=1e-5)
    assert int(st) == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, kv_heads, size, pairs, norm", [
    (4, 2, 16, 4, "head"), (3, 1, 24, 12, "row"), (8, 1, 64, 16, "row"), (6, 6, 64, 0, "head"), (5, 5, 40, 20, "row"),
    (2, 2, 256, 0, "row"), (1, 1, 8, 4, "head"), (24, 8, 16, 8, "row"), (12, 2, 128, 32, "row"), (14, 2, 64, 32, "head"),
])
@pytest.mark.parametrize("values", ["keys", "projected"])
@pytest.mark.parametrize("splits", [1, 3])
@pytest.mark.parametrize("tokens", [23, 150])
def test_store_with_weighted_norms_and_values_from_keys(dev, dtype, heads, kv_heads, size, pairs, norm, values, splits,
                                                        tokens):
    """A few rows and partial sums take the kernel of a warp per head; 150 rows of bfloat16 whose sizes
    are multiples of eight take the kernel of 16-byte pieces."""
    from einf_b200 import ops

    gen = torch.Generator().manual_seed(3)
    page_size, pages, value_size = 4, tokens // 4 + 4, size if values == "keys" else 24
    width = (heads + kv_heads) * size + (0 if values == "keys" else kv_heads * value_size)
    if splits == 1:
        qkv = torch.randn((tokens, width), generator=gen).to(dtype).to(dev)
    else:
        qkv = torch.randn((splits, tokens, width), generator=gen).to(dev)
    rows = norm == "row"
    q_weight = (1 + 0.3 * torch.randn(heads * size if rows else size, generator=gen)).to(dev)
    k_weight = (1 + 0.3 * torch.randn(kv_heads * size if rows else size, generator=gen)).to(dev)
    slots = torch.randperm(pages * page_size, generator=gen)[:tokens].to(torch.int32).to(dev)
    slots[5] = -1
    positions = torch.randint(0, 500, (tokens,), generator=gen).to(torch.int32).to(dev)
    inv_freq = (10000.0 ** (-torch.arange(pairs).float() / max(pairs, 1))).to(dev) if pairs else None
    results = []
    for fn in (ops.qkv_norm_store, ref.qkv_norm_store):
        q_out = torch.zeros((tokens, heads, size), dtype=dtype, device=dev)
        k_cache = torch.zeros((pages, kv_heads, page_size, size), dtype=dtype, device=dev)
        v_cache = torch.zeros((pages, kv_heads, page_size, value_size), dtype=dtype, device=dev)
        st = status(dev)
        fn(qkv, None, slots, q_out, k_cache, v_cache, heads, kv_heads, size, value_size, 1e-5, st, positions=positions,
           inv_freq=inv_freq, q_norm_weight=q_weight, k_norm_weight=k_weight, norm_rows=rows,
           values_from_keys=values == "keys")
        assert int(st) == 0
        results.append((q_out, k_cache, v_cache))
    for got, want in zip(*results):
        torch.testing.assert_close(got, want, **(dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else tol(dtype)))
    if values == "keys" and splits == 1:
        # the cached values are the projected keys themselves, untouched by norm, weight and rotation
        keep = slots >= 0
        page, offset = (slots[keep] // page_size).long(), (slots[keep] % page_size).long()
        raw = qkv[:, heads * size:].reshape(tokens, kv_heads, size)[keep]
        assert torch.equal(results[0][2][page, :, offset, :], raw)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, kv_heads, size, page_size", [
    (4, 2, 16, 4), (8, 1, 64, 16), (6, 2, 48, 16), (3, 3, 128, 16), (40, 8, 32, 8),
])
@pytest.mark.parametrize("window", [None, 5])
def test_general_attention_with_a_sink(dev, dtype, heads, kv_heads, size, page_size, window):
    from einf_b200 import ops

    requests = [(0, 1), (0, 2 * page_size), (3, 6), (15, 6), (page_size * 4 - 1, 1), (70, 1), (0, 37)]
    (q, k, v, table, seq, pos), scale, window = _attention_case(dev, dtype, heads, kv_heads, size, page_size, requests, window)
    sink = (torch.randn(heads, generator=torch.Generator().manual_seed(1)) * 3).to(dev)
    sink[0] = 40.0          # larger than any score: nearly all of head 0's weight
    sink[-1] = -40.0        # as good as absent
    st = status(dev)
    out = torch.full((q.shape[0], heads, size), float("nan"), dtype=dtype, device=dev)
    ops.paged_attention_generic(q, k, v, table, seq, pos, out, scale, window, st, sink=sink)
    want = torch.empty_like(out)
    ref.paged_attention_generic(q, k, v, table, seq, pos, want, scale, window, st, sink=sink)
    plain = torch.empty_like(out)
    ref.paged_attention_generic(q, k, v, table, seq, pos, plain, scale, window, st)
    assert int(st) == 0
    torch.testing.assert_close(out, want, **(dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else tol(dtype)))
    torch.testing.assert_close(out[:, -1], plain[:, -1], **(dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else tol(dtype)))
    assert float(out[:, 0].float().abs().max()) < 1e-3 * float(plain[:, 0].float().abs().max()) + 1e-3


@pytest.mark.parametrize("experts, top, groups", [
    (12, 4, (2, 1)), (12, 4, (3, 2)), (9, 3, (3, 1)), (8, 8, (4, 4)), (64, 6, (8, 3)), (5, 2, None), (1, 1, (1, 1)),
    (160, 8, (40, 5)),
])
@pytest.mark.parametrize("score", ["softmax", "sigmoid"])
def test_router_with_a_correction_and_groups(dev, experts, top, groups, score):
    from einf_b200 import ops

    gen = torch.Generator().manual_seed(7)
    tokens, width = 41, experts + 3          # the row holds three columns that are not the router's
    logits = (torch.randn((tokens, width), generator=gen) * 2).to(dev)
    correction = (torch.randn(experts, generator=gen) * 0.2 - 0.1).to(dev)     # mostly negative choice scores count too
    results = []
    for fn in (ops.router_topk, ref.router_topk):
        ids = torch.zeros((tokens, top), dtype=torch.int32, device=dev)
        weights = torch.zeros((tokens, top), dtype=torch.float32, device=dev)
        fn(logits, top, score, False, ids, weights, experts, correction, groups)
        results.append((ids, weights))
    assert torch.equal(results[0][0], results[1][0])
    torch.testing.assert_close(results[0][1], results[1][1], rtol=1e-5, atol=1e-7)
    if groups is not None:
        per = experts // groups[0]
        for row in results[0][0].cpu().tolist():
            assert len({e // per for e in row}) <= groups[1] and len(set(row)) == top
    # the weights are the scores, without the correction
    z = logits[:, :experts]
    scores = torch.softmax(z, dim=-1) if score == "softmax" else torch.sigmoid(z)
    torch.testing.assert_close(results[0][1], torch.gather(scores, 1, results[0][0].long()), rtol=1e-5, atol=1e-7)
    # the same logits as three partial sums
    parts = torch.stack([logits * 0.5, logits * 0.25, logits * 0.25])
    ids = torch.zeros((tokens, top), dtype=torch.int32, device=dev)
    weights = torch.zeros((tokens, top), dtype=torch.float32, device=dev)
    ops.router_topk(parts, top, score, False, ids, weights, experts, correction, groups)
    assert torch.equal(ids, results[1][0])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens, hidden, experts, identity, top", [(1, 32, 4, 2, 3), (50, 48, 6, 3, 4), (300, 200, 3, 1, 2),
                                                                   (17, 40, 1, 1, 2), (9, 64, 5, 0, 2)])
def test_combine_with_pass_through_experts_and_a_gated_addend(dev, dtype, tokens, hidden, experts, identity, top):
    from einf_b200 import ops

    gen = torch.Generator().manual_seed(11)
    outputs = experts + identity
    ids = torch.stack([torch.randperm(outputs, generator=gen)[:top] for _ in range(tokens)]).to(torch.int32).to(dev)
    weights = torch.rand((tokens, top), generator=gen).to(dev)
    x = torch.randn((tokens, hidden), generator=gen).to(dtype).to(dev)
    work = torch.empty((3 * experts + 1,), dtype=torch.int32, device=dev)
    place = torch.zeros((tokens, top), dtype=torch.int32, device=dev)
    sorted_x = torch.zeros((tokens * top, hidden), dtype=dtype, device=dev)
    ops.moe_dispatch(x, ids, weights, experts, False, work, place, sorted_x)
    y = torch.randn((tokens * top, hidden), generator=gen).to(dtype).to(dev)
    addend = torch.randn((2, tokens, hidden), generator=gen).to(dev)                 # split-K partial sums
    gate = torch.randn((3, tokens, outputs + 1), generator=gen).to(dev)
    out = torch.empty((tokens, hidden), dtype=torch.float32, device=dev)
    ops.moe_combine(y, ids, place, weights, True, addend, out, experts, identity_input=x, num_identity=identity,
                    addend_gate=(gate, outputs))
    # stated from the pairs themselves
    want = addend.sum(0) * torch.sigmoid(gate.sum(0)[:, outputs])[:, None]
    for j in range(top):
        e = ids[:, j].long()
        routed = weights[:, j, None] * y.float()[place[:, j].long()]
        through = weights[:, j, None] * x.float()
        want = want + torch.where((e < experts)[:, None], routed, through)
    torch.testing.assert_close(out, want, rtol=1e-5, atol=1e-5)
    again = torch.empty_like(out)
    ref.moe_combine(y, ids, place, weights, True, addend, again, experts, identity_input=x, num_identity=identity,
                    addend_gate=(gate, outputs))
    torch.testing.assert_close(again, want, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, dim, vdim, cap", [(2, 48, 48, 15.0), (1, 16, 8, 4.0), (3, 8, 20, 30.0), (4, 64, 64, 15.0),
                                                  (2, 128, 12, 1.0)])
@pytest.mark.parametrize("portions", [(1, 1, 1), (7, 1, 30, 2), (300,), (130, 129, 1), (1100,), (257, 600)])
def test_matrix_memory_steps(dev, dtype, heads, dim, vdim, cap, portions):
    """Gates, recurrence on the widened values and output, chained as the mixer chains them, against
    the plain statements; then the same tokens in two steps, which must carry maximum and state."""
    from einf_b200 import ops

    gen = torch.Generator().manual_seed(13)
    requests = len(portions)
    tokens = sum(portions)
    columns = ops.memory_value_columns(vdim)
    assert columns % 4 == 0 and columns > vdim
    q_start = torch.tensor([0] + list(torch.tensor(portions).cumsum(0)), dtype=torch.int32, device=dev)
    slots = torch.tensor([2, 0, 3, 1][:requests], dtype=torch.int32, device=dev)
    slots[-1] = -1 if requests > 2 else slots[-1]          # a request without a slot starts from zero, stores nothing
    row = heads * dim * columns + heads
    raw = (torch.randn((tokens, 2 * heads), generator=gen) * 6).to(dev)
    bias = torch.randn(2 * heads, generator=gen).to(dev)
    proj = (torch.randn((tokens, 2 * heads * dim + 2 * heads * vdim), generator=gen) * 0.7).to(dtype).to(dev)
    keys = heads * dim
    q, k = proj[:, :keys], proj[:, keys:2 * keys]
    v, gate = proj[:, 2 * keys:2 * keys + heads * vdim], proj[:, 2 * keys + heads * vdim:]
    weight = (1 + 0.2 * torch.randn(heads * vdim, generator=gen)).to(dev)
    start_state = torch.randn((4, row), generator=gen).to(dev) * 0.3

    def run(module, state, first, last, starts, step_slots, longest):
        n = last - first
        decay, scale, floor = (torch.empty((n, heads), dtype=torch.float32, device=dev) for _ in range(3))
        wide = torch.empty((n, heads * columns), dtype=dtype, device=dev)
        memory = state[:, :heads * dim * columns].view(4, heads, dim, columns)
        top = state[:, heads * dim * columns:]
        module.memory_gates(raw[first:last], bias, cap, v[first:last], top, starts, step_slots, decay, scale, floor, wide,
                            heads, vdim)
        # single tokens of a few requests: the kernel's CTAs share a head's rows and leave parts of y
        parts = module.recurrence_step_splits(step_slots.shape[0], heads, dim, columns, memory) if longest == 1 else 1
        y = torch.empty((n, heads * columns) if parts == 1 else (parts, n, heads * columns), dtype=torch.float32, device=dev)
        module.linear_recurrence(q[first:last], k[first:last], wide, memory, starts, step_slots, y, heads, heads, dim,
                                 columns, token_decay=decay, token_scale=scale, max_q_len=longest)
        out = torch.empty((n, heads * vdim), dtype=dtype, device=dev)
        module.memory_output(y, floor, gate[first:last], weight, out, heads, vdim, dim ** -0.5, 1e-5, 1e-6)
        return out, (decay, scale, floor, wide)

    state_ops, state_ref = start_state.clone(), start_state.clone()
    got, parts = run(ops, state_ops, 0, tokens, q_start, slots, max(portions))
    want, parts_ref = run(ref, state_ref, 0, tokens, q_start, slots, max(portions))
    for a, b in zip(parts, parts_ref):
        torch.testing.assert_close(a.float(), b.float(), rtol=2e-5, atol=1e-6)
    assert float(parts[0].max()) <= 1.0 and float(parts[1].max()) <= 1.0
    close = dict(rtol=3e-4, atol=3e-4) if dtype == torch.float32 else tol(dtype)
    torch.testing.assert_close(got.float(), want.float(), **close)
    torch.testing.assert_close(state_ops, state_ref, rtol=3e-4, atol=3e-4)
    if requests == 1 and portions[0] > 2:
        # the same request in two steps: 2 tokens short of the whole, then the rest
        cut = portions[0] - 2
        state_two = start_state.clone()
        one = torch.tensor([0, cut], dtype=torch.int32, device=dev)
        two = torch.tensor([0, 2], dtype=torch.int32, device=dev)
        head, _ = run(ops, state_two, 0, cut, one, slots, cut)
        tail, _ = run(ops, state_two, cut, tokens, two, slots, 2)
        torch.testing.assert_close(torch.cat([head, tail]).float(), got.float(), **close)
        torch.testing.assert_close(state_two, state_ops, rtol=3e-4, atol=3e-4)


@pytest.mark.parametrize("widths", [(48,), (200,), (1536,), (5000,)])
@pytest.mark.parametrize("kinds", [("f32", "bf16"), ("split", "f32"), ("bf16",), ("split", "split", "f32", "bf16")])
@pytest.mark.parametrize("tokens", [19, 300])
def test_normed_join_of_branches(dev, widths, kinds, tokens):
    from einf_b200 import ops

    gen = torch.Generator().manual_seed(17)
    width = widths[0]
    terms, weights = [], []
    for index, kind in enumerate(kinds):
        if kind == "split":
            terms.append(torch.randn((3, tokens, width), generator=gen).to(dev) * (index + 1))
        else:
            dtype = torch.float32 if kind == "f32" else torch.bfloat16
            terms.append((torch.randn((tokens, width), generator=gen) * (index + 1)).to(dtype).to(dev))
        weights.append((1 + 0.2 * torch.randn(width, generator=gen)).to(dev))
    out = torch.empty((tokens, width), dtype=torch.float32, device=dev)
    ops.norm_join(terms, weights, 1e-5, out, 0.5)
    want = torch.zeros_like(out)
    for term, weight in zip(terms, weights):
        t = term.float().sum(0) if term.dim() == 3 else term.float()
        want += weight * t / torch.sqrt(t.pow(2).mean(-1, keepdim=True) + 1e-5)
    torch.testing.assert_close(out, 0.5 * want, rtol=2e-5, atol=2e-5)
    again = torch.empty_like(out)
    ref.norm_join(terms, weights, 1e-5, again, 0.5)
    torch.testing.assert_close(again, 0.5 * want, rtol=2e-5, atol=2e-5)


@pytest.mark.parametrize("heads, kv_heads, size, page_size", [(8, 1, 64, 16), (14, 2, 64, 16), (12, 2, 128, 16),
                                                             (4, 4, 128, 32), (40, 2, 64, 8)])
@pytest.mark.parametrize("window", [None, 150])
def test_tensor_core_attention_with_a_sink(dev, heads, kv_heads, size, page_size, window):
    """The tcgen05 kernels for prompt portions and for single tokens, side by side in one step, with a
    sink per head: one CTA per row tile, clusters that share a row tile's keys, clusters that share
    a single token's keys and several clusters per token."""
    from einf_b200 import ops
    from test_kanavik_kernels import _step_split

    dtype = torch.bfloat16
    requests = [(0, 1), (0, 2 * page_size), (3, 6), (page_size * 4 - 1, 1), (700, 1), (0, 300), (2100, 64), (5000, 1)]
    (q, k, v, table, seq, pos), scale, window = _attention_case(dev, dtype, heads, kv_heads, size, page_size, requests, window)
    sink = (torch.randn(heads, generator=torch.Generator().manual_seed(2)) * 3).to(dev)
    sink[0], sink[-1] = 40.0, -40.0
    q_tiles, singles = _step_split(requests)
    st = status(dev)
    want = torch.empty((q.shape[0], heads, size), dtype=dtype, device=dev)
    ref.paged_attention_generic(q, k, v, table, seq, pos, want, scale, window, st, sink=sink)
    longest = max(s + n for s, n in requests)
    for cluster in (0, 1, 4):
        out = torch.full_like(want, float("nan"))
        ops.paged_prefill_attention(q, k, v, table, q_tiles.to(dev), out, scale, window, st, prefill_cluster=cluster,
                                    cached_before=2100, sink=sink)
        ops.paged_decode_attention_auto(q, k, v, table, seq, pos, out, scale, window, st, singles.to(dev),
                                        max_context=longest, sink=sink)
        assert int(st) == 0
        torch.testing.assert_close(out, want, **tol(dtype))
    for cluster, splits in ((1, 1), (8, 1), (16, 1), (4, 3)):
        out = torch.full_like(want, float("nan"))
        ops.paged_decode_attention_tcgen05(q, k, v, table, seq, pos, out, scale, window, cluster, st, singles.to(dev),
                                           splits, sink=sink)
        assert int(st) == 0
        rows = singles.long().to(dev)
        torch.testing.assert_close(out[rows], want[rows], **tol(dtype))
