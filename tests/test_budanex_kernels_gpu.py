"""The kernels of the Budanex mixers alone against plain functions, on inputs made so that a
fault shows: one key whose score stands out placed just inside and just outside a window, at page
borders and far back; a sink that outweighs every key; soft caps that bite; convolution state
shorter than the taps; recurrent state carried over cuts of every size."""
import math

import pytest
import torch

import plain_budanex as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def _tol(dtype):
    return 2e-5 if dtype == torch.float32 else 2e-2


def _paged(k, v, dtype, ring=0):
    """One sequence's keys and values written into pages in a scrambled order."""
    n, g, d = k.shape
    dv = v.shape[-1]
    n_pages = (n + 63) // 64 if not ring else ring // 64
    order = list(reversed(range(n_pages)))
    kc = torch.zeros((n_pages + 1, g, 64, d), dtype=dtype, device=DEV)
    vc = torch.zeros((n_pages + 1, g, 64, dv), dtype=dtype, device=DEV)
    lo = max(0, n - ring) if ring else 0
    for j in range(lo, n):
        p_eff = j % ring if ring else j
        page = order[p_eff // 64]
        kc[page, :, p_eff % 64] = k[j].to(dtype)
        vc[page, :, p_eff % 64] = v[j].to(dtype)
    table = torch.tensor(order, dtype=torch.int32, device=DEV)
    return kc, vc, table


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window, standout", [
    (0, 3), (70, 0), (70, 1), (64, 0), (64, 1), (65, 0), (1, 0), (136, 0), (136, 1), (200, 150)])
def test_attention_kernel_with_a_key_that_stands_out(dtype, window, standout):
    """600 keys; for the query at position 599 one key's score is far above the others.
    ``standout`` counts from the oldest key the window admits: 0 is the last one inside (for a
    causal run, position 3: far back); the key one further back (outside) stands out as well,
    with another value, so a window that is one off changes the result completely."""
    from minfer_b200.kernels import api as K
    torch.manual_seed(window * 7 + standout)
    n, H, G, D, Dv = 600, 4, 2, 24, 40
    q = torch.randn(n, H, D, dtype=torch.float64) * 0.5
    k = torch.randn(n, G, D, dtype=torch.float64) * 0.5
    v = torch.randn(n, G, Dv, dtype=torch.float64)
    last = n - 1
    inside = (last - window + 1 + standout) if window else standout
    marked = [inside] + ([inside - 1] if window and standout == 0 and inside >= 1 else [])
    for h in range(H):
        for j in marked:
            k[j, h // 2] = q[last, h // 2 * 2] * 3.0
    for j in marked:
        v[j] = 10.0 * (1 + marked.index(j))
    q, k, v = (t.to(dtype).to(torch.float64) for t in (q, k, v))
    sink = torch.tensor([0.3, -1.0, 2.0, 0.0], dtype=torch.float64)
    rows = [last, last - 1, 64, 63, 0]
    want = P.scored_attention(q[rows], k, v, rows, 0.4, window, 25.0, sink)
    qd = q[rows].to(dtype).to(DEV).contiguous()
    row_seq = torch.zeros(len(rows), dtype=torch.int32, device=DEV)
    row_pos = torch.tensor(rows, dtype=torch.int32, device=DEV)
    cu = torch.tensor([0, n], dtype=torch.int32, device=DEV)
    sink_d = sink.to(torch.float32).to(DEV)
    out = torch.empty((len(rows), H * Dv), dtype=dtype, device=DEV)
    K.sink_attention_packed(qd, k.to(dtype).to(DEV), v.to(dtype).to(DEV), row_seq, row_pos, cu, out,
                            None, None, H, G, D, Dv, window, 0, True, 0.4, sink_logit=sink_d,
                            softcap=25.0)
    err = float((out.cpu().to(torch.float64).view(len(rows), H, Dv) - want).abs().max())
    assert err < _tol(dtype) * float(want.abs().max()), err
    for ring in ([0] if not window else [0, ((window + 63) // 64) * 64 + 64]):
        kc, vc, table = _paged(k, v, dtype, ring)
        live = [r for r in rows if not ring or r > last - (ring - window + 1)]
        sel = [rows.index(r) for r in live]
        out2 = torch.empty((len(live), H * Dv), dtype=dtype, device=DEV)
        K.sink_attention_paged(qd[sel].contiguous(), kc, vc, row_seq[:len(live)].contiguous(),
                               row_pos[sel].contiguous(), table, table.numel(), ring, out2, None,
                               None, H, G, D, Dv, window, 0, True, 0.4, sink_logit=sink_d,
                               softcap=25.0)
        err = float((out2.cpu().to(torch.float64).view(len(live), H, Dv) - want[sel]).abs().max())
        assert err < _tol(dtype) * float(want.abs().max()), (ring, err)
        if dtype != torch.bfloat16:
            continue
        # the tensor-core kernels: single queries over the pages ...
        out3 = torch.empty((len(live), H * Dv), dtype=dtype, device=DEV)
        K.sink_attention_decode(qd[sel].contiguous(), kc, vc, row_seq[:len(live)].contiguous(),
                                row_pos[sel].contiguous(), table, table.numel(), ring, out3, None,
                                None, H, G, D, Dv, window, 0, True, 0.4, window if window else n,
                                sink_logit=sink_d, softcap=25.0)
        err = float((out3.cpu().to(torch.float64).view(len(live), H, Dv) - want[sel]).abs().max())
        assert err < _tol(dtype) * float(want.abs().max()), ("decode", ring, err)
        # ... and the sequence's last 50 tokens as one portion over the pages
        tail = list(range(n - 50, n))
        want_tail = P.scored_attention(q[tail], k, v, tail, 0.4, window, 25.0, sink)
        out4 = torch.empty((50, H * Dv), dtype=dtype, device=DEV)
        K.sink_attention_mma(q[tail].to(dtype).to(DEV).contiguous(), kc, vc,
                             torch.tensor([0, 50], dtype=torch.int32, device=DEV),
                             torch.tensor([n], dtype=torch.int32, device=DEV), table, table.numel(),
                             ring, out4, None, None, 1, 50, H, G, D, Dv, window, 0, True, 0.4,
                             sink_logit=sink_d, softcap=25.0)
        err = float((out4.cpu().to(torch.float64).view(50, H, Dv) - want_tail).abs().max())
        assert err < _tol(dtype) * float(want.abs().max()), ("portion", ring, err)
    if dtype == torch.bfloat16:
        # the whole prompt over its own packed keys on tensor cores
        out5 = torch.empty((n, H * Dv), dtype=dtype, device=DEV)
        K.sink_attention_mma(q.to(dtype).to(DEV).contiguous(), k.to(dtype).to(DEV), v.to(dtype).to(DEV),
                             cu, None, None, 0, 0, out5, None, None, 1, n, H, G, D, Dv, window, 0,
                             True, 0.4, sink_logit=sink_d, softcap=25.0)
        err = float((out5[rows].cpu().to(torch.float64).view(len(rows), H, Dv) - want).abs().max())
        assert err < _tol(dtype) * float(want.abs().max()), ("prompt", err)


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_sink_that_outweighs_the_keys_and_a_cap_that_bites(dtype):
    from minfer_b200.kernels import api as K
    torch.manual_seed(5)
    n, H, D, Dv = 90, 3, 16, 8
    q = (torch.randn(n, H, D, dtype=torch.float64) * 2).to(dtype).to(torch.float64)
    k = (torch.randn(n, 1, D, dtype=torch.float64) * 2).to(dtype).to(torch.float64)
    v = torch.randn(n, 1, Dv, dtype=torch.float64).to(dtype).to(torch.float64)
    rows = list(range(n))
    cu = torch.tensor([0, n], dtype=torch.int32, device=DEV)
    pos = torch.arange(n, dtype=torch.int32, device=DEV)
    seq = torch.zeros(n, dtype=torch.int32, device=DEV)
    for sink, cap in ((torch.tensor([6.0, 0.0, -4.0]), 2.0), (None, 1.0), (torch.tensor([9.0] * 3), 0.0)):
        want = P.scored_attention(q, k, v, rows, 1.0, 0, cap,
                                  None if sink is None else sink.to(torch.float64))
        out = torch.empty((n, H * Dv), dtype=dtype, device=DEV)
        K.sink_attention_packed(q.to(dtype).to(DEV), k.to(dtype).to(DEV), v.to(dtype).to(DEV), seq, pos,
                                cu, out, None, None, H, 1, D, Dv, 0, 0, sink is not None, 1.0,
                                sink_logit=None if sink is None else sink.to(DEV), softcap=cap)
        err = float((out.cpu().to(torch.float64).view(n, H, Dv) - want).abs().max())
        assert err < _tol(dtype) * max(1.0, float(want.abs().max())), (cap, err)


@pytest.mark.parametrize("sizes", [(3, 20, 1, 28, 18, 8, 12, 18, 18, 5),      # multiples of nothing
                                   (3, 24, 2, 32, 20, 8, 16, 24, 40, 8),      # of 4: 16-byte accesses
                                   (2, 64, 1, 128, 96, 32, 32, 96, 96, 0)])
@pytest.mark.parametrize("style", ["half", "interleaved"])
@pytest.mark.parametrize("dtype", DTYPES)
def test_prepare_kernel_norms_rotates_and_writes_pages(dtype, style, sizes):
    """Whole-segment norms with weights, a rotation of part of each head from an offset, values
    that are the key's first elements, and the cache pages, against plain functions."""
    from minfer_b200.kernels import api as K
    torch.manual_seed(11)
    n = 70
    H, qw, G, kw, vw, rot, q_off_rot, k_off_rot, k_norm_n, slack = sizes
    width = H * qw + G * kw + slack
    proj = torch.randn(n, width, dtype=torch.float64)
    positions = list(range(1990, 1990 + n))            # large angles
    qn = 1 + 0.1 * torch.randn(H * qw, dtype=torch.float64)
    kn = 1 + 0.1 * torch.randn(k_norm_n, dtype=torch.float64)  # the first elements of the key segment
    freqs = P.plain_frequencies(rot, 10000.0)
    mag = 1.25
    qs = P.rms_norm(proj[:, :H * qw], qn, 1e-5).view(n, H, qw).clone()
    ks = proj[:, H * qw:H * qw + G * kw].clone()
    ks[:, :k_norm_n] = P.rms_norm(ks[:, :k_norm_n], kn, 1e-5)
    ks = ks.view(n, G, kw)
    qs[:, :, q_off_rot:q_off_rot + rot] = P.rotate(qs[:, :, q_off_rot:q_off_rot + rot].contiguous(),
                                                   positions, freqs, style, mag)
    ks[:, :, k_off_rot:k_off_rot + rot] = P.rotate(ks[:, :, k_off_rot:k_off_rot + rot].contiguous(),
                                                   positions, freqs, style, mag)
    q_out = torch.empty((n, H, qw), dtype=dtype, device=DEV)
    k_out = torch.empty((n, G, kw), dtype=dtype, device=DEV)
    v_out = torch.empty((n, G, vw), dtype=dtype, device=DEV)
    n_pages = (1990 + n + 63) // 64
    kc = torch.zeros((n_pages, G, 64, kw), dtype=dtype, device=DEV)
    vc = torch.zeros((n_pages, G, 64, vw), dtype=dtype, device=DEV)
    table = torch.arange(n_pages, dtype=torch.int32, device=DEV).flip(0).contiguous()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    K.qk_prepare(proj.to(torch.float32).to(DEV), torch.tensor(positions, dtype=torch.int32, device=DEV),
                 torch.zeros(n, dtype=torch.int32, device=DEV),
                 torch.tensor([1990 + n], dtype=torch.int32, device=DEV), q_out, k_out, v_out, kc, vc,
                 table, n_pages, 0, q_off=0, n_heads=H, q_width=qw, k_off=H * qw, n_kv=G, k_width=kw,
                 v_off=0, v_width=vw, v_from_k=True, q_norm=qn.to(torch.float32).to(DEV),
                 k_norm=kn.to(torch.float32).to(DEV), eps=1e-5,
                 inv_freq=torch.tensor(freqs, dtype=torch.float64, device=DEV), rot_dims=rot,
                 rot_style=0 if style == "half" else 1, rot_magnitude=mag, q_rot_off=q_off_rot,
                 k_rot_off=k_off_rot, status=status)
    tol = 3e-5 if dtype == torch.float32 else 2e-2
    assert float((q_out.cpu().double() - qs).abs().max()) < tol * float(qs.abs().max())
    assert float((k_out.cpu().double() - ks).abs().max()) < tol * float(ks.abs().max())
    assert float((v_out.cpu().double() - ks[:, :, :vw]).abs().max()) < tol * float(ks.abs().max())
    for i, p in enumerate(positions):
        page = int(table[p // 64])
        assert torch.equal(kc[page, :, p % 64], k_out[i]) and torch.equal(vc[page, :, p % 64], v_out[i])
    assert int(status.item()) == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_per_head_products_with_gate_and_tail(dtype):
    from minfer_b200.kernels import api as K
    torch.manual_seed(3)
    n, H, J, D, tail = 45, 3, 37, 21, 6
    x = torch.randn(n, H * (D + tail) + 2, dtype=torch.float64).to(dtype)
    w = (torch.randn(H, J, D, dtype=torch.float64) * 0.3).to(dtype)
    gate = torch.randn(n, H * J + 9, dtype=torch.float32)
    xh = x[:, :H * (D + tail)].double().view(n, H, D + tail)
    want = torch.einsum("hjd,nhd->nhj", w.double(), xh[:, :, :D])
    y = torch.empty((n, H * (J + tail)), dtype=dtype, device=DEV)
    K.head_linear(x.to(DEV), w.to(DEV), y, x_head=D + tail, x_off=0, y_head=J + tail, tail=tail,
                  x_tail_off=D)
    got = y.cpu().double().view(n, H, J + tail)
    tol = 2e-5 if dtype == torch.float32 else 1.5e-2
    assert float((got[:, :, :J] - want).abs().max()) < tol * float(want.abs().max())
    assert torch.equal(got[:, :, J:], xh[:, :, D:])
    y2 = torch.empty((n, H * J), dtype=dtype, device=DEV)
    K.head_linear(x.to(DEV), w.to(DEV), y2, x_head=D + tail, x_off=0, y_head=J, gate=gate.to(DEV),
                  gate_off=9)
    want2 = want * torch.sigmoid(gate[:, 9:].double().view(n, H, J))
    assert float((y2.cpu().double().view(n, H, J) - want2).abs().max()) < tol * float(want.abs().max())


def _mamba_setup(seed, heads, P_, N, groups, taps, norm_groups, width=48):
    torch.manual_seed(seed)
    inner = heads * P_
    ch = inner + 2 * groups * N
    w = {"in": torch.randn(2 * inner + 2 * groups * N + heads, width, dtype=torch.float64) * 0.2,
         "conv": torch.randn(ch, taps, dtype=torch.float64) * 0.4,
         "conv.b": torch.randn(ch, dtype=torch.float64) * 0.1,
         "dt_bias": torch.randn(heads, dtype=torch.float64) * 0.5 - 1.0,
         # slow decay in some heads: what a far token wrote is still there hundreds later
         "A_log": torch.linspace(-4.0, 0.5, heads, dtype=torch.float64),
         "D": torch.randn(heads, dtype=torch.float64),
         "norm": 1 + 0.1 * torch.randn(inner, dtype=torch.float64),
         "o": torch.randn(width, inner, dtype=torch.float64) * 0.2}
    m = {"heads": heads, "vdim": P_, "state": N, "groups": groups, "conv": taps,
         "norm_groups": norm_groups}
    return w, m


@pytest.mark.parametrize("sizes", [(4, 8, 16, 2, 4, 2), (3, 20, 24, 1, 3, 1), (6, 5, 7, 6, 1, 3),
                                   (2, 70, 130, 2, 8, 4), (8, 64, 128, 1, 4, 1), (2, 16, 256, 1, 2, 1)])
@pytest.mark.parametrize("cuts", [[200], [1] * 40, [2] * 30, [3, 1, 2, 64, 65, 1, 7], [150, 2, 1, 1, 46]])
def test_state_space_kernels_over_cuts(sizes, cuts):
    """Convolution, recurrence and gated norm as the mixer chains them, a sequence fed in cuts of
    every size (shorter than the taps too), beside a second sequence in another slot, against the
    plain mixer over the whole sequence."""
    from minfer_b200.kernels import api as K
    heads, P_, N, groups, taps, norm_groups = sizes
    w, m = _mamba_setup(sum(sizes), heads, P_, N, groups, taps, norm_groups)
    inner, ch = heads * P_, heads * P_ + 2 * groups * N
    n = sum(cuts)
    u = torch.randn(n, 48, dtype=torch.float64)
    u2 = torch.randn(n, 48, dtype=torch.float64)
    wp = {"mix." + k_: v_ for k_, v_ in w.items()}
    want = [P.mamba2_mixer(x, wp, "mix.", m, 1e-5) for x in (u, u2)]
    f32 = lambda t: t.to(torch.float32).to(DEV).contiguous()
    ssm = torch.zeros((5, heads, P_, N), dtype=torch.float32, device=DEV)
    conv = torch.zeros((5, ch, taps - 1), dtype=torch.float32, device=DEV)
    ssm[1].fill_(7.0)                                   # a slot nobody uses keeps what it holds
    slots = torch.tensor([3, 0], dtype=torch.int32, device=DEV)
    got = [[], []]
    at = 0
    for c in cuts:
        xs = torch.cat([u[at:at + c], u2[at:at + c]])
        proj = f32(xs @ w["in"].T)
        token_row = torch.tensor([0] * c + [1] * c, dtype=torch.int32, device=DEV)
        cu = torch.tensor([0, c, 2 * c], dtype=torch.int32, device=DEV)
        uc = torch.empty((2 * c, ch), dtype=torch.float32, device=DEV)
        K.conv_silu(proj, inner, ch, f32(w["conv"]), f32(w["conv.b"]), conv, token_row, cu, slots, uc,
                    2, single=(c == 1))
        y = torch.empty((2 * c, inner), dtype=torch.float32, device=DEV)
        K.ssm_scan(uc, proj, inner + ch, f32(w["dt_bias"]), f32(w["A_log"]), f32(w["D"]), ssm, cu, slots,
                   y, 2, heads, P_, N, groups)
        g = torch.empty((2 * c, inner), dtype=torch.float32, device=DEV)
        K.gated_group_norm(y, proj, 0, f32(w["norm"]), g, norm_groups, 1e-5)
        out = g.cpu().double() @ w["o"].T
        got[0].append(out[:c])
        got[1].append(out[c:])
        at += c
    for r in range(2):
        err = float((torch.cat(got[r]) - want[r]).abs().max())
        assert err < 3e-5 * float(want[r].abs().max()), (r, err)
    assert float(ssm[1].min()) == 7.0 and float(ssm[2].abs().max()) == 0.0


@pytest.mark.parametrize("activation", ["silu", "gelu_tanh"])
def test_gated_activation_kernels(activation):
    from minfer_b200.kernels import api as K
    from minfer_b200.kernels import gemm
    torch.manual_seed(2)
    n, width, ff = 70, 64, 136
    x = (torch.randn(n, width) * 2).to(torch.bfloat16)
    g = (torch.randn(ff, width) * 0.3).to(torch.bfloat16)
    u = (torch.randn(ff, width) * 0.3).to(torch.bfloat16)
    act = P.gelu_tanh if activation == "gelu_tanh" else P.silu
    want = act(x.double() @ g.double().T) * (x.double() @ u.double().T)
    gu = torch.cat([x.double() @ g.double().T, x.double() @ u.double().T], dim=1).to(torch.float32).to(DEV)
    out = torch.empty((n, ff), dtype=torch.float32, device=DEV)
    K.swiglu(gu, out, False, activation)
    assert float((out.cpu().double() - want).abs().max()) < 1e-5 * float(want.abs().max())
    packed = torch.stack([g, u], dim=1).reshape(2 * ff, width).contiguous().to(DEV)
    out16 = torch.empty((n, ff), dtype=torch.bfloat16, device=DEV)
    K.gemm_tc(x.to(DEV), packed, None, out16, K.gated_epilogue(activation), gemm.status_word(torch.device(DEV)))
    assert float((out16.cpu().double() - want).abs().max()) < 1e-2 * float(want.abs().max())


def test_soft_cap_and_stream_add():
    from minfer_b200.kernels import api as K
    torch.manual_seed(9)
    x = torch.randn(33, 130) * 40
    d = x.to(DEV)
    K.tanh_cap(d, 15.0)
    assert float((d.cpu().double() - 15.0 * torch.tanh(x.double() / 15.0)).abs().max()) < 1e-5
    h = torch.randn(20, 72)
    e = torch.randn(20, 72)
    v = torch.randn(72).to(torch.bfloat16)
    hd = h.to(DEV)
    K.add_stream(hd, e.to(DEV), v.to(DEV))
    assert torch.allclose(hd.cpu(), h + e + v.float(), atol=1e-6)
    hd = h.to(DEV)
    K.add_stream(hd, None, v.float().to(DEV))
    assert torch.allclose(hd.cpu(), h + v.float(), atol=1e-6)


@pytest.mark.parametrize("heads, kv", [(40, 1), (34, 2), (16, 1), (17, 1)])
def test_single_queries_with_many_heads_on_one_key_head(heads, kv):
    """The tensor-core kernel for single queries takes a key/value head's query heads in blocks
    of 16: groups of 40, 17 (a block of one head) and exactly 16."""
    from minfer_b200.kernels import api as K
    torch.manual_seed(heads)
    n, D, Dv, window = 300, 32, 16, 150
    dtype = torch.bfloat16
    q = (torch.randn(n, heads, D, dtype=torch.float64) * 0.7).to(dtype).double()
    k = (torch.randn(n, kv, D, dtype=torch.float64) * 0.7).to(dtype).double()
    v = torch.randn(n, kv, Dv, dtype=torch.float64).to(dtype).double()
    sink = torch.linspace(-2.0, 2.0, heads, dtype=torch.float64)
    rows = [n - 1, 200, 149, 150, 3]
    want = P.scored_attention(q[rows], k, v, rows, 0.3, window, 0.0, sink)
    kc, vc, table = _paged(k, v, dtype)
    out = torch.empty((len(rows), heads * Dv), dtype=dtype, device=DEV)
    K.sink_attention_decode(q[rows].to(dtype).to(DEV).contiguous(), kc, vc,
                            torch.zeros(len(rows), dtype=torch.int32, device=DEV),
                            torch.tensor(rows, dtype=torch.int32, device=DEV), table, table.numel(), 0,
                            out, None, None, heads, kv, D, Dv, window, 0, True, 0.3, window,
                            sink_logit=sink.float().to(DEV))
    err = float((out.cpu().double().view(len(rows), heads, Dv) - want).abs().max())
    assert err < 2e-2 * float(want.abs().max()), err
