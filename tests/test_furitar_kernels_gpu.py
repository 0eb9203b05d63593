"""Each kernel of the Furitar parts alone, against the plain functions of ``plain_furitar``:
norm + token shift with its state, the xIELU activation, learned positions, the unit norm of
q and k with the cache write, and the attention with its changed scores, chunk mask and sink,
over packed keys and over pages, in float32 and bfloat16.  Where random inputs would hide a
fault (one key far back among hundreds, the keys at a chunk's edge, the sink), a query and a key
are scaled so that one score stands out."""
import pytest
import torch

import plain_furitar as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 3e-6, "bfloat16": 1.2e-2}


def K():
    from minfer_b200.kernels import api
    return api


def _i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def _err(got, want):
    got, want = got.detach().double().cpu(), want.detach().double().cpu()
    return float((got - want).abs().max() / max(1e-30, float(want.abs().max())))


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width", [72, 100, 517, 2048])
def test_norm_and_shift_with_state(dtype, width):
    """Three sequences in one step: one starts at position 0, one goes on with several tokens,
    one with a single token; then a second step goes on from the state the first left."""
    g = torch.Generator().manual_seed(width)
    counts, starts, slots = [5, 3, 1], [0, 7, 2], [4, 0, 2]
    n = sum(counts)
    x = torch.randn(n, width, generator=g).to(DEV)
    w = (1 + 0.1 * torch.randn(width, generator=g)).to(DEV)
    s = (0.5 + 0.4 * torch.randn(width, generator=g)).to(DEV)
    state = torch.randn(6, width, generator=g).to(DEV)
    state0 = state.clone()
    cu = [0, 5, 8, 9]
    positions = [p for c, st in zip(counts, starts) for p in range(st, st + c)]
    token_row = [b for b, c in enumerate(counts) for _ in range(c)]
    out = torch.empty(n, width, dtype=DT[dtype], device=DEV)
    K().norm_shift(x, w, s, 1e-5, _i32(positions), _i32(token_row), _i32(cu), _i32(slots), state, out,
                   multi=True)
    xd, wd, sd = x.double().cpu(), w.double().cpu(), s.double().cpu()
    for b in range(3):
        h = P.rms_norm(xd[cu[b]:cu[b + 1]], wd, 1e-5)
        before = state0[slots[b]].double().cpu() if starts[b] > 0 else torch.zeros(width, dtype=torch.float64)
        want = P.token_shift(h, before, sd)
        assert _err(out[cu[b]:cu[b + 1]], want) < TOL[dtype]
        assert _err(state[slots[b]], h[-1]) < 3e-6            # the state is float32 in both
    for untouched in (1, 3, 5):
        assert torch.equal(state[untouched], state0[untouched])
    # one token each, from the state just written
    x2 = torch.randn(3, width, generator=g).to(DEV)
    state1 = state.clone()
    out2 = torch.empty(3, width, dtype=DT[dtype], device=DEV)
    K().norm_shift(x2, w, s, 1e-5, _i32([5, 10, 3]), _i32([0, 1, 2]), _i32([0, 1, 2, 3]), _i32(slots),
                   state, out2, multi=False)
    for b in range(3):
        h = P.rms_norm(x2[b:b + 1].double().cpu(), wd, 1e-5)
        want = P.token_shift(h, state1[slots[b]].double().cpu(), sd)
        assert _err(out2[b:b + 1], want) < TOL[dtype]
        assert _err(state[slots[b]], h[-1]) < 3e-6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_norm_and_shift_adds_pending_splits(dtype):
    """One token a row: the K splits of the projection before are added into x by the kernel."""
    g = torch.Generator().manual_seed(21)
    width, rows = 136, 4
    x = torch.randn(rows, width, generator=g).to(DEV)
    parts = torch.randn(3, rows, width, generator=g).to(DEV)
    bias = torch.randn(width, generator=g).to(DEV)
    w = (1 + 0.1 * torch.randn(width, generator=g)).to(DEV)
    s = (0.5 + 0.4 * torch.randn(width, generator=g)).to(DEV)
    state = torch.randn(5, width, generator=g).to(DEV)
    state0 = state.clone()
    full = x.double().cpu() + parts.double().cpu().sum(0) + bias.double().cpu()
    out = torch.empty(rows, width, dtype=DT[dtype], device=DEV)
    K().norm_shift(x, w, s, 1e-5, _i32([3, 0, 9, 1]), _i32([0, 1, 2, 3]), _i32([0, 1, 2, 3, 4]),
                   _i32([2, 0, 4, 1]), state, out, multi=False, partial=parts, bias=bias)
    assert _err(x, full) < 3e-6                           # x is complete in memory afterwards
    for b, (slot, pos) in enumerate(zip([2, 0, 4, 1], [3, 0, 9, 1])):
        h = P.rms_norm(full[b:b + 1], w.double().cpu(), 1e-5)
        before = state0[slot].double().cpu() if pos > 0 else torch.zeros(width, dtype=torch.float64)
        assert _err(out[b:b + 1], P.token_shift(h, before, s.double().cpu())) < TOL[dtype]
        assert _err(state[slot], h[-1]) < 3e-6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_xielu(dtype):
    g = torch.Generator().manual_seed(1)
    z = (3 * torch.randn(37, 129, generator=g)).to(DEV)
    z[0, :4] = torch.tensor([0.0, -0.0, 1e-4, -1e-4])
    for a in ([0.3, -0.7], [-2.0, 1.5], [0.0, 0.0]):
        params = torch.tensor(a, dtype=torch.float32, device=DEV)
        out = torch.empty(37, 129, dtype=DT[dtype], device=DEV)
        K().xielu(z, params, out)
        want = P.xielu(z.double().cpu(), params.double().cpu())
        assert _err(out, want) < TOL[dtype]


@pytest.mark.parametrize("table_dtype", ["float32", "bfloat16"])
def test_learned_positions_are_added_by_position(table_dtype):
    g = torch.Generator().manual_seed(2)
    table = torch.randn(50, 72, generator=g).to(DT[table_dtype]).to(DEV)
    h = torch.randn(6, 72, generator=g).to(DEV)
    h0 = h.clone()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    pos = [0, 1, 49, 7, 7, 30]
    K().add_rows(h, table, _i32(pos), status)
    assert torch.allclose(h, h0 + table[pos].float(), rtol=0, atol=1e-6)
    assert int(status.item()) == 0
    K().add_rows(h, table, _i32([0, 1, 50, 7, 7, 30]), status)       # outside the table
    assert int(status.item()) & 2


# ---------------------------------------------------------------------------------------------
def _qkv_case(seed, n_heads, n_kv, hd, vd, lengths):
    g = torch.Generator().manual_seed(seed)
    n = sum(lengths)
    q = P.rms_unit(torch.randn(n, n_heads, hd, generator=g, dtype=torch.float64), 1e-6)
    k = P.rms_unit(torch.randn(n, n_kv, hd, generator=g, dtype=torch.float64), 1e-6)
    v = torch.randn(n, n_kv, vd, generator=g, dtype=torch.float64)
    r1 = 0.5 + 0.3 * torch.rand(n_heads, generator=g, dtype=torch.float64)
    r2 = 0.2 + torch.rand(n_heads, generator=g, dtype=torch.float64)
    return q, k, v, r1, r2


def _plain_rows(q, k, v, r1, r2, scale, chunk, lengths):
    outs, at = [], 0
    for n in lengths:
        sl = slice(at, at + n)
        outs.append(P.sink_attention(q[sl], k[sl], v[sl], list(range(n)), list(range(n)), r1, r2,
                                     scale, chunk))
        at += n
    return torch.cat(outs).reshape(q.shape[0], -1)


def _spike(q, k, v, lengths, chunk, group):
    """In every sequence, for the query at the last position i of the sequence: the key at its
    chunk's first position and the key just before that chunk are turned into large multiples
    of the query, and their values into +-100: what leaks from outside the chunk shows, what
    is lost inside shows, and a far key among hundreds carries the answer."""
    at = 0
    for n in lengths:
        i = n - 1
        lo = (i // chunk) * chunk if chunk > 0 else 0
        for h_kv in range(k.shape[1]):
            qd = q[at + i, h_kv * group]
            k[at + lo, h_kv] = 3.0 * qd
            v[at + lo, h_kv] = 100.0
            if lo > 0:
                k[at + lo - 1, h_kv] = 4.0 * qd
                v[at + lo - 1, h_kv] = -100.0
        at += n


CASES = [  # heads, kv, hd, vd, chunk, lengths
    (4, 2, 16, 24, 10, [23, 1, 40]),
    (6, 3, 20, 12, 64, [130, 64, 65]),
    (3, 3, 12, 20, 1, [5, 9]),
    (2, 1, 24, 40, 0, [300, 17]),
    (8, 2, 64, 64, 200, [401, 200, 201]),
    (16, 1, 64, 128, 150, [310]),
    (4, 4, 128, 128, 128, [129, 257]),
    (5, 1, 256, 256, 7, [30]),
]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("bias, sink", [(True, True), (False, True), (True, False)])
def test_attention_over_packed_keys(dtype, case, bias, sink):
    heads, kv, hd, vd, chunk, lengths = case
    q, k, v, r1, r2 = _qkv_case(hd + vd, heads, kv, hd, vd, lengths)
    _spike(q, k, v, lengths, chunk, heads // kv)
    if not bias:
        r1 = r2 = torch.zeros(heads, dtype=torch.float64)
    t = DT[dtype]
    qd, kd, vd_ = q.to(t).to(DEV), k.to(t).to(DEV), v.to(t).to(DEV)
    want = _plain_rows(qd.double().cpu(), kd.double().cpu(), vd_.double().cpu(), r1, r2, 0.3, chunk, lengths)
    if not sink:          # the plain function always has the sink: take it out of the weights
        no_sink = _plain_rows(qd.double().cpu(), kd.double().cpu(), torch.ones_like(vd_).double().cpu(), r1,
                              r2, 0.3, chunk, lengths)       # = 1 - weight of the sink, per head
        want = (want.view(-1, heads, vd) / no_sink.view(-1, heads, vd)[..., :1]).reshape(want.shape)
    cu = [0]
    for n in lengths:
        cu.append(cu[-1] + n)
    row_seq = [b for b, n in enumerate(lengths) for _ in range(n)]
    row_pos = [p for n in lengths for p in range(n)]
    out = torch.empty(sum(lengths), heads * vd, dtype=t, device=DEV)
    f = lambda x: x.float().to(DEV) if bias else None
    K().sink_attention_packed(qd, kd, vd_, _i32(row_seq), _i32(row_pos), _i32(cu), out, f(r1), f(r2),
                              heads, kv, hd, vd, 0, chunk, sink, 0.3)
    assert _err(out, want) < (2e-5 if dtype == "float32" else 1.5e-2)


def _paged(k, v, lengths, ring, seed):
    """Lays packed keys and values out in pages behind a shuffled page table (ring > 0: at
    position % ring, only the last ``ring`` positions of a sequence)."""
    n_kv, hd, vd = k.shape[1], k.shape[2], v.shape[2]
    per_seq = [min(-(-n // 64), ring // 64) if ring else -(-n // 64) for n in lengths]
    total = sum(per_seq) + 3
    perm = torch.randperm(total, generator=torch.Generator().manual_seed(seed)).tolist()
    kc = torch.full((total, n_kv, 64, hd), 7.0, dtype=k.dtype)      # other pages hold rubbish
    vc = torch.full((total, n_kv, 64, vd), -9.0, dtype=v.dtype)
    stride = max(per_seq)
    table = torch.full((len(lengths), stride), -1, dtype=torch.int32)
    at, used = 0, 0
    for b, n in enumerate(lengths):
        for i in range(per_seq[b]):
            table[b, i] = perm[used]
            used += 1
        for p in range(max(0, n - ring) if ring else 0, n):
            pe = p % ring if ring else p
            page = int(table[b, pe // 64])
            kc[page, :, p % 64] = k[at + p]
            vc[page, :, p % 64] = v[at + p]
        at += n
    return kc, vc, table, stride


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("ringed", [False, True])
def test_attention_over_pages(dtype, case, ringed):
    """The last positions of every sequence as queries over the paged cache, linear and ring."""
    heads, kv, hd, vd, chunk, lengths = case
    if ringed and chunk == 0:
        pytest.skip("a ring needs a bound on how far a query looks back")
    q, k, v, r1, r2 = _qkv_case(3 * hd + vd, heads, kv, hd, vd, lengths)
    _spike(q, k, v, lengths, chunk, heads // kv)
    t = DT[dtype]
    qd, kd, vd_ = q.to(t), k.to(t), v.to(t)
    want_all = _plain_rows(qd.double(), kd.double(), vd_.double(), r1, r2, 0.3, chunk, lengths)
    ring = -(-(chunk + 20) // 64) * 64 if ringed else 0
    kc, vc, table, stride = _paged(kd, vd_, lengths, ring, seed=hd)
    rows, row_seq, row_pos, at = [], [], [], 0
    for b, n in enumerate(lengths):
        tail = min(n, 21 if ring else n)           # a ring serves the positions a step may add
        for p in range(n - tail, n):
            rows.append(at + p)
            row_seq.append(b)
            row_pos.append(p)
        at += n
    out = torch.empty(len(rows), heads * vd, dtype=t, device=DEV)
    K().sink_attention_paged(qd[rows].contiguous().to(DEV), kc.to(DEV), vc.to(DEV), _i32(row_seq),
                             _i32(row_pos), table.reshape(-1).to(DEV), stride, ring, out,
                             r1.float().to(DEV), r2.float().to(DEV), heads, kv, hd, vd, 0, chunk, True, 0.3)
    assert _err(out, want_all[rows]) < (2e-5 if dtype == "float32" else 1.5e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("splits", [0, 3])
def test_unit_norm_and_cache_write(dtype, splits):
    """q and k come out with unit root mean square per head, v unchanged; all three land in the
    step's packed tensors and in the right places of the right pages."""
    heads, kv, hd, vd = 4, 2, 20, 12
    lengths, starts = [70, 3], [0, 126]
    g = torch.Generator().manual_seed(9)
    n = sum(lengths)
    width = (heads + kv) * hd + kv * vd
    full = torch.randn(n, width, generator=g)
    if splits:
        parts = torch.randn(splits, n, width, generator=g)
        parts[0] = full - parts[1:].sum(0)
        qkv = parts.to(DEV)
    else:
        qkv = full.to(DEV)
    t = DT[dtype]
    table = _i32([[5, 2, -1], [0, 4, 1]])
    kc = torch.zeros(6, kv, 64, hd, dtype=t, device=DEV)
    vc = torch.zeros(6, kv, 64, vd, dtype=t, device=DEV)
    positions = [p for c, s in zip(lengths, starts) for p in range(s, s + c)]
    token_row = [b for b, c in enumerate(lengths) for _ in range(c)]
    q_out = torch.empty(n, heads, hd, dtype=t, device=DEV)
    k_out = torch.empty(n, kv, hd, dtype=t, device=DEV)
    v_out = torch.empty(n, kv, vd, dtype=t, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    K().unit_norm_kvstore(qkv, _i32(positions), _i32(token_row), _i32([70, 129]), q_out, k_out, v_out,
                          kc, vc, table.reshape(-1), 3, 0, heads, kv, hd, vd, 1e-5, True, status,
                          n_partials=splits)
    fd = full.double()
    q = P.rms_unit(fd[:, :heads * hd].view(n, heads, hd), 1e-5)
    k = P.rms_unit(fd[:, heads * hd:(heads + kv) * hd].view(n, kv, hd), 1e-5)
    v = fd[:, (heads + kv) * hd:].view(n, kv, vd)
    tol = 1e-5 if dtype == "float32" else 8e-3
    assert _err(q_out, q) < tol and _err(k_out, k) < tol and _err(v_out, v) < tol
    assert int(status.item()) == 0
    pages = [[5, 2], [0, 4, 1]]
    for i, (b, p) in enumerate(zip(token_row, positions)):
        page = pages[b][p // 64]
        assert torch.equal(kc[page, :, p % 64], k_out[i]) and torch.equal(vc[page, :, p % 64], v_out[i])
    assert float(kc[3].abs().max()) == 0.0 and float(kc[2, :, 6:].abs().max()) == 0.0


# ---------------------------------------------------------------------------------------------
# the tensor-core kernels (bfloat16)
# ---------------------------------------------------------------------------------------------
MMA_CASES = [  # heads, kv, hd, vd, chunk, lengths
    (8, 2, 64, 64, 200, [401, 200, 201, 1]),
    (16, 1, 64, 128, 150, [310, 64]),
    (4, 4, 128, 128, 128, [129, 257]),
    (6, 2, 48, 72, 88, [333, 87, 89]),
    (2, 1, 128, 40, 64, [191]),
    (4, 2, 8, 8, 1, [70]),
    (3, 1, 104, 56, 0, [500, 17]),
    (4, 2, 64, 64, 5000, [300]),
]


@pytest.mark.parametrize("case", MMA_CASES)
@pytest.mark.parametrize("bias, sink", [(True, True), (False, True), (True, False)])
def test_prompt_kernel_on_tensor_cores_packed(case, bias, sink):
    heads, kv, hd, vd, chunk, lengths = case
    q, k, v, r1, r2 = _qkv_case(hd + 2 * vd, heads, kv, hd, vd, lengths)
    _spike(q, k, v, lengths, chunk, heads // kv)
    if not bias:
        r1 = r2 = torch.zeros(heads, dtype=torch.float64)
    t = torch.bfloat16
    qd, kd, vd_ = q.to(t).to(DEV), k.to(t).to(DEV), v.to(t).to(DEV)
    want = _plain_rows(qd.double().cpu(), kd.double().cpu(), vd_.double().cpu(), r1, r2, 0.3, chunk, lengths)
    if not sink:
        ones = _plain_rows(qd.double().cpu(), kd.double().cpu(), torch.ones_like(vd_).double().cpu(), r1,
                           r2, 0.3, chunk, lengths)
        want = (want.view(-1, heads, vd) / ones.view(-1, heads, vd)[..., :1]).reshape(want.shape)
    cu = [0]
    for n in lengths:
        cu.append(cu[-1] + n)
    out = torch.empty(sum(lengths), heads * vd, dtype=t, device=DEV)
    f = lambda x: x.float().to(DEV) if bias else None
    assert K().sink_attention_mma_supported(t, hd, vd)
    K().sink_attention_mma(qd, kd, vd_, _i32(cu), None, None, 0, 0, out, f(r1), f(r2), len(lengths),
                           max(lengths), heads, kv, hd, vd, 0, chunk, sink, 0.3)
    assert _err(out, want) < 2e-2


@pytest.mark.parametrize("case", MMA_CASES)
@pytest.mark.parametrize("ringed", [False, True])
def test_prompt_kernel_on_tensor_cores_over_pages(case, ringed):
    """The last positions of every sequence as one step's rows over the paged cache."""
    heads, kv, hd, vd, chunk, lengths = case
    if ringed and (chunk == 0 or chunk > 1000):
        pytest.skip("a ring needs a bound on how far a query looks back")
    q, k, v, r1, r2 = _qkv_case(5 * hd + vd, heads, kv, hd, vd, lengths)
    _spike(q, k, v, lengths, chunk, heads // kv)
    t = torch.bfloat16
    qd, kd, vd_ = q.to(t), k.to(t), v.to(t)
    want_all = _plain_rows(qd.double(), kd.double(), vd_.double(), r1, r2, 0.3, chunk, lengths)
    tail_max = 70
    ring = -(-(chunk + tail_max - 1) // 64) * 64 if ringed else 0
    kc, vc, table, stride = _paged(kd, vd_, lengths, ring, seed=vd)
    rows, cu, at = [], [0], 0
    for n in lengths:
        tail = min(n, tail_max)
        rows += list(range(at + n - tail, at + n))
        cu.append(cu[-1] + tail)
        at += n
    out = torch.empty(len(rows), heads * vd, dtype=t, device=DEV)
    K().sink_attention_mma(qd[rows].contiguous().to(DEV), kc.to(DEV), vc.to(DEV), _i32(cu),
                           _i32(lengths), table.reshape(-1).to(DEV), stride, ring, out,
                           r1.float().to(DEV), r2.float().to(DEV), len(lengths), tail_max, heads, kv,
                           hd, vd, 0, chunk, True, 0.3)
    assert _err(out, want_all[rows]) < 2e-2


def test_xielu_in_the_products_epilogue():
    """The up projection with the activation in its epilogue against product, then activation."""
    g = torch.Generator().manual_seed(4)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for m, n, k in ((5, 136, 72), (64, 256, 256), (300, 384, 128), (1000, 512, 264)):
        x = torch.randn(m, k, generator=g).to(torch.bfloat16).to(DEV)
        w = (0.2 * torch.randn(n, k, generator=g)).to(torch.bfloat16).to(DEV)
        a = torch.tensor([0.4, -0.3], dtype=torch.float64)
        sp = P.softplus(a)
        for out_dtype in (torch.bfloat16, torch.float32):
            out = torch.empty(m, n, dtype=out_dtype, device=DEV)
            K().gemm_tc_xielu(x, w, out, float(sp[0]), 0.5 + float(sp[1]), status)
            want = P.xielu(x.double().cpu() @ w.double().cpu().T, a)
            assert _err(out, want) < (1.2e-2 if out_dtype == torch.bfloat16 else 2e-4)
    assert int(status.item()) == 0


@pytest.mark.parametrize("case", MMA_CASES)
@pytest.mark.parametrize("ringed", [False, True])
@pytest.mark.parametrize("sink", [True, False])
def test_single_query_kernel_on_tensor_cores(case, ringed, sink):
    """The last positions of every sequence, each a query of its own, over the paged cache."""
    heads, kv, hd, vd, chunk, lengths = case
    if ringed and (chunk == 0 or chunk > 1000):
        pytest.skip("a ring needs a bound on how far a query looks back")
    if heads // kv > 16:
        pytest.skip("more query heads per key/value head than the product has rows")
    q, k, v, r1, r2 = _qkv_case(7 * hd + vd, heads, kv, hd, vd, lengths)
    _spike(q, k, v, lengths, chunk, heads // kv)
    t = torch.bfloat16
    qd, kd, vd_ = q.to(t), k.to(t), v.to(t)
    want_all = _plain_rows(qd.double(), kd.double(), vd_.double(), r1, r2, 0.3, chunk, lengths)
    if not sink:
        ones = _plain_rows(qd.double(), kd.double(), torch.ones_like(vd_).double(), r1, r2, 0.3, chunk, lengths)
        want_all = (want_all.view(-1, heads, vd) / ones.view(-1, heads, vd)[..., :1]).reshape(want_all.shape)
    ring = -(-(chunk + 20) // 64) * 64 if ringed else 0
    kc, vc, table, stride = _paged(kd, vd_, lengths, ring, seed=hd + 1)
    rows, row_seq, row_pos, at = [], [], [], 0
    for b, n in enumerate(lengths):
        tail = min(n, 21 if ring else 40)
        for p in list(range(n - tail, n)) + ([0] if not ring else []):
            rows.append(at + p)
            row_seq.append(b)
            row_pos.append(p)
        at += n
    out = torch.empty(len(rows), heads * vd, dtype=t, device=DEV)
    reach = chunk if chunk > 0 else max(lengths)
    K().sink_attention_decode(qd[rows].contiguous().to(DEV), kc.to(DEV), vc.to(DEV), _i32(row_seq),
                              _i32(row_pos), table.reshape(-1).to(DEV), stride, ring, out,
                              r1.float().to(DEV), r2.float().to(DEV), heads, kv, hd, vd, 0, chunk, sink,
                              0.3, reach)
    assert _err(out, want_all[rows]) < 2e-2
    # one query alone: the plan cuts its keys into many splits, which the merge kernel adds up
    one = [len(rows) - 1]
    out1 = torch.empty(1, heads * vd, dtype=t, device=DEV)
    K().sink_attention_decode(qd[rows][one].contiguous().to(DEV), kc.to(DEV), vc.to(DEV),
                              _i32([row_seq[-1]]), _i32([row_pos[-1]]), table.reshape(-1).to(DEV),
                              stride, ring, out1, r1.float().to(DEV), r2.float().to(DEV), heads, kv, hd,
                              vd, 0, chunk, sink, 0.3, reach)
    assert _err(out1, want_all[[rows[-1]]]) < 2e-2


TC_CASES = [  # heads, kv, hd, chunk, lengths   (keys and values of one size, 64 or 128)
    (8, 2, 64, 200, [401, 200, 201, 1]),
    (4, 4, 128, 128, [129, 257, 600]),
    (4, 2, 64, 5000, [300]),
    (2, 1, 128, 0, [700, 17]),
    (2, 2, 64, 1, [70]),
    (6, 3, 128, 88, [333, 87, 89]),
]


@pytest.mark.parametrize("case", TC_CASES)
@pytest.mark.parametrize("bias, sink", [(True, True), (False, True), (True, False)])
def test_prompt_kernel_tcgen05_packed(case, bias, sink):
    heads, kv, hd, chunk, lengths = case
    q, k, v, r1, r2 = _qkv_case(11 * hd, heads, kv, hd, hd, lengths)
    _spike(q, k, v, lengths, chunk, heads // kv)
    if not bias:
        r1 = r2 = torch.zeros(heads, dtype=torch.float64)
    t = torch.bfloat16
    qd, kd, vd_ = q.to(t).to(DEV), k.to(t).to(DEV), v.to(t).to(DEV)
    want = _plain_rows(qd.double().cpu(), kd.double().cpu(), vd_.double().cpu(), r1, r2, 0.3, chunk, lengths)
    if not sink:
        ones = _plain_rows(qd.double().cpu(), kd.double().cpu(), torch.ones_like(vd_).double().cpu(), r1,
                           r2, 0.3, chunk, lengths)
        want = (want.view(-1, heads, hd) / ones.view(-1, heads, hd)[..., :1]).reshape(want.shape)
    cu = [0]
    for n in lengths:
        cu.append(cu[-1] + n)
    out = torch.empty(sum(lengths), heads * hd, dtype=t, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    f = lambda x: x.float().to(DEV) if bias else None
    K().sink_attention_tc(qd, kd, vd_, _i32(cu), None, None, 0, 0, out, f(r1), f(r2), len(lengths),
                          max(lengths), heads, kv, hd, 0, chunk, sink, 0.3, status)
    assert int(status.item()) == 0
    assert _err(out, want) < 2e-2


@pytest.mark.parametrize("case", TC_CASES)
@pytest.mark.parametrize("ringed", [False, True])
def test_prompt_kernel_tcgen05_over_pages(case, ringed):
    heads, kv, hd, chunk, lengths = case
    if ringed and (chunk == 0 or chunk > 1000):
        pytest.skip("a ring needs a bound on how far a query looks back")
    q, k, v, r1, r2 = _qkv_case(13 * hd, heads, kv, hd, hd, lengths)
    _spike(q, k, v, lengths, chunk, heads // kv)
    t = torch.bfloat16
    qd, kd, vd_ = q.to(t), k.to(t), v.to(t)
    want_all = _plain_rows(qd.double(), kd.double(), vd_.double(), r1, r2, 0.3, chunk, lengths)
    tail_max = 170
    ring = -(-(chunk + tail_max - 1) // 64) * 64 if ringed else 0
    kc, vc, table, stride = _paged(kd, vd_, lengths, ring, seed=hd + 3)
    rows, cu, at = [], [0], 0
    for n in lengths:
        tail = min(n, tail_max)
        rows += list(range(at + n - tail, at + n))
        cu.append(cu[-1] + tail)
        at += n
    out = torch.empty(len(rows), heads * hd, dtype=t, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    K().sink_attention_tc(qd[rows].contiguous().to(DEV), kc.to(DEV), vc.to(DEV), _i32(cu), _i32(lengths),
                          table.reshape(-1).to(DEV), stride, ring, out, r1.float().to(DEV),
                          r2.float().to(DEV), len(lengths), tail_max, heads, kv, hd, 0, chunk, True, 0.3,
                          status)
    assert int(status.item()) == 0
    assert _err(out, want_all[rows]) < 2e-2


@pytest.mark.parametrize("table_dtype", ["float32", "bfloat16"])
def test_embedding_adds_position_rows_itself(table_dtype):
    g = torch.Generator().manual_seed(8)
    t = DT[table_dtype]
    table = torch.randn(40, 72, generator=g).to(t).to(DEV)
    rows = torch.randn(50, 72, generator=g).to(t).to(DEV)
    ids, pos = [3, 39, 0, 7], [0, 49, 12, 12]
    out = torch.empty(4, 72, dtype=torch.float32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    K().embed(table, _i32(ids), out, status, 1.7, rows=rows, row_index=_i32(pos))
    want = table[ids].float() * 1.7 + rows[pos].float()
    assert torch.equal(out, want) and int(status.item()) == 0
    K().embed(table, _i32(ids), out, status, 1.7, rows=rows, row_index=_i32([0, 50, 12, 12]))
    assert int(status.item()) & 2 and torch.equal(out[1], table[39].float() * 1.7)
