"""Each kernel alone against a plain PyTorch reference of the same operation (fp64 on the
host), at sizes other than the engine's: widths and vocabularies that are no power of two,
head sizes in steps of 16, odd head and group counts."""
import math

import numpy as np
import pytest
import torch

import plain_lfm2 as P

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def dev(t, dtype=None):
    return t.to(device=DEV, dtype=dtype or t.dtype).contiguous()


def close(got, want, rel, what=""):
    got = got.detach().double().cpu()
    want = want.detach().double().cpu()
    assert got.shape == want.shape, f"{what}: {got.shape} vs {want.shape}"
    scale = max(1.0, want.abs().max().item())
    err = (got - want).abs().max().item()
    assert math.isfinite(err) and err <= rel * scale, f"{what}: max|delta| {err:.3e} > {rel:.1e}*{scale:.3g}"


@pytest.fixture(autouse=True)
def guard_bands():
    """Every test of this file runs with canaries around the outputs its kernels allocate."""
    from gpu_util import GuardedOutputs
    with GuardedOutputs() as guard:
        yield guard
        guard.check()
        guard.forget()


def bf16_round(t):
    return t.to(torch.bfloat16).to(t.dtype)


# ------------------------------------------------------------------ elementwise
@pytest.mark.parametrize("V,H,T", [(300, 100, 7), (1000, 72, 1), (17, 2048, 33)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed(V, H, T, dtype):
    from flyweight_b200.kernels import ops
    g = torch.Generator().manual_seed(0)
    table = torch.randn(V, H, generator=g).to(dtype)
    ids = torch.randint(0, V, (T,), generator=g, dtype=torch.int32)
    out = ops.embed(dev(table), dev(ids))
    assert out.dtype == torch.float32
    assert torch.equal(out.cpu(), table.float()[ids.long()])


@pytest.mark.parametrize("H", [64, 100, 1000, 2048, 4100])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_with_and_without_the_residual_sum(H, out_dtype):
    from flyweight_b200.kernels import ops
    g = torch.Generator().manual_seed(H)
    x = torch.randn(9, H, generator=g) * 3
    d = torch.randn(9, H, generator=g)
    w = 1 + 0.1 * torch.randn(H, generator=g)
    eps = 1e-5
    tol = 1e-5 if out_dtype == torch.float32 else 2.0 ** -8

    def ref(v):
        v = v.double()
        return v * torch.rsqrt((v * v).mean(-1, keepdim=True) + eps) * w.double()

    xd = dev(x)
    close(ops.rmsnorm(xd, dev(w), eps, out_dtype), ref(x), tol, "norm")
    assert torch.equal(xd.cpu(), x)
    out = ops.rmsnorm(xd, dev(w), eps, out_dtype, delta=dev(d))
    close(out, ref(x + d), tol, "sum + norm")
    assert torch.equal(xd.cpu(), x + d)                       # the sum is stored, in fp32
    rows = torch.tensor([5, 0, 5, 8], dtype=torch.int32)
    xd = dev(x)
    out = ops.rmsnorm(xd, dev(w), eps, out_dtype, delta=dev(d), rows=dev(rows))
    close(out, ref(x + d)[rows.long()], tol, "gathered sum + norm")
    assert torch.equal(xd.cpu(), x)                           # a gather leaves x alone


@pytest.mark.parametrize("T,F", [(1, 192), (5, 320), (130, 1000)])
def test_silu_mul(T, F):
    from flyweight_b200.kernels import ops
    g = torch.Generator().manual_seed(1)
    gu = torch.randn(T, 2 * F, generator=g) * 4
    want = torch.from_numpy(P.silu(gu[:, :F].double().numpy())) * gu[:, F:].double()
    close(ops.silu_mul(dev(gu), torch.float32), want, 1e-6, "silu fp32")
    gb = gu.to(torch.bfloat16)
    want = torch.from_numpy(P.silu(gb[:, :F].double().numpy())) * gb[:, F:].double()
    close(ops.silu_mul(dev(gb), torch.bfloat16), want, 2.0 ** -8, "silu bf16")
    big = torch.tensor([[100.0, -100.0, 1.0, 1.0]])
    out = ops.silu_mul(dev(big), torch.float32).cpu()
    assert torch.isfinite(out).all() and abs(out[0, 0].item() - 100.0) < 1e-4 and out[0, 1].abs() < 1e-30


# ------------------------------------------------------------------ matrix products
@pytest.mark.parametrize("M,N,K", [(1, 1, 1), (3, 70, 50), (65, 129, 17), (130, 384, 96), (8, 100, 333)])
def test_gemm_simt_fp32(M, N, K):
    from flyweight_b200.kernels import ops
    g = torch.Generator().manual_seed(M * N + K)
    x, w = torch.randn(M, K, generator=g), torch.randn(N, K, generator=g)
    add = torch.randn(M, N, generator=g)
    close(ops.gemm_simt(dev(x), dev(w), torch.float32), x.double() @ w.double().T, 1e-6, "gemm")
    close(ops.gemm_simt(dev(x), dev(w), torch.float32, addend=dev(add)),
          x.double() @ w.double().T + add.double(), 1e-6, "gemm + addend")


def test_gemm_row_does_not_depend_on_the_batch():
    from flyweight_b200.kernels import ops
    g = torch.Generator().manual_seed(5)
    x, w = torch.randn(70, 200, generator=g), torch.randn(90, 200, generator=g)
    whole = ops.gemm_simt(dev(x), dev(w), torch.float32)
    single = ops.gemm_simt(dev(x[41:42]), dev(w), torch.float32)
    assert torch.equal(whole[41:42], single)


@pytest.mark.parametrize("M,N,K", [(1, 64, 64), (9, 200, 96), (200, 320, 96), (64, 2048, 512),
                                   (300, 1000, 264), (128, 256, 2048)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_linear_bf16(M, N, K, out_dtype):
    """The product the bfloat16 path uses, whichever kernel the dispatcher picks."""
    from flyweight_b200.kernels import ops
    g = torch.Generator().manual_seed(M + N + K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    want = x.double() @ w.double().T
    tol = 1e-5 if out_dtype == torch.float32 else 2.0 ** -8
    close(ops.linear(dev(x), dev(w), out_dtype), want, tol, f"linear {M}x{N}x{K}")
    if out_dtype == torch.float32:
        add = torch.randn(M, N, generator=g)
        close(ops.linear(dev(x), dev(w), out_dtype, addend=dev(add)), want + add.double(), 1e-5,
              "linear + addend")


# ------------------------------------------------------------------ gated short convolution
def conv_reference(p, taps, bias, state, segments):
    """Token by token with a rolling state per slot (float64)."""
    T, H3 = p.shape
    H = H3 // 3
    L = taps.shape[1]
    z = torch.zeros(T, H, dtype=torch.float64)
    state = state.clone().double()
    t = 0
    for slot, n in segments:
        for _ in range(n):
            b, c, x = p[t, :H].double(), p[t, H:2 * H].double(), p[t, 2 * H:].double()
            window = torch.cat([state[slot], (b * x)[:, None]], dim=1)
            state[slot] = window[:, 1:]
            y = (window * taps.double()).sum(1)
            if bias is not None:
                y = y + bias.double()
            z[t] = c * y
            t += 1
    return z, state


@pytest.mark.parametrize("H,L,bias", [(64, 3, False), (96, 4, True), (100, 2, True), (40, 7, False)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_shortconv_over_ragged_segments(H, L, bias, dtype):
    from flyweight_b200.kernels import ops
    g = torch.Generator().manual_seed(H + L)
    segments = [(2, 1), (0, 5), (3, 1), (1, 2), (4, L - 1), (5, 40), (6, 1)]   # (slot, tokens)
    T = sum(n for _, n in segments)
    p = torch.randn(T, 3 * H, generator=g).to(dtype)
    taps = torch.randn(H, L, generator=g)
    b = torch.randn(H, generator=g) if bias else None
    state = torch.randn(8, H, L - 1, generator=g)
    seg_start = torch.tensor(np.cumsum([0] + [n for _, n in segments]), dtype=torch.int32)
    seg_slot = torch.tensor([s for s, _ in segments], dtype=torch.int32)
    tok_seg = torch.tensor([i for i, (_, n) in enumerate(segments) for _ in range(n)], dtype=torch.int32)
    want_z, want_state = conv_reference(p, taps, b, state, segments)
    sd = dev(state)
    z = ops.shortconv(dev(p), dev(taps), None if b is None else dev(b), sd, dev(seg_start),
                      dev(seg_slot), dev(tok_seg), len(segments), dtype)
    tol = 1e-5 if dtype == torch.float32 else 2.0 ** -7
    close(z, want_z, tol, "conv output")
    close(sd, want_state, 1e-6, "conv state")
    assert torch.equal(sd[7].cpu(), state[7])                 # an unused slot is untouched


@pytest.mark.parametrize("H,L,bias", [(64, 3, True), (104, 2, False), (72, 4, True), (40, 5, False)])
def test_shortconv_prompt_sized_bfloat16(H, L, bias):
    """Long segments take the kernel that slides a window over runs of tokens: segment edges
    inside a run, a run that starts at a segment's first tokens, the tail of the batch."""
    from flyweight_b200.kernels import ops
    g = torch.Generator().manual_seed(H * L)
    segments = [(1, 130), (0, 1), (2, 2), (3, 301), (4, L - 1), (5, 67), (6, 3)]
    T = sum(n for _, n in segments)
    p = torch.randn(T, 3 * H, generator=g).to(torch.bfloat16)
    taps = torch.randn(H, L, generator=g)
    b = torch.randn(H, generator=g) if bias else None
    state = torch.randn(8, H, L - 1, generator=g)
    seg_start = torch.tensor(np.cumsum([0] + [n for _, n in segments]), dtype=torch.int32)
    seg_slot = torch.tensor([s for s, _ in segments], dtype=torch.int32)
    tok_seg = torch.tensor([i for i, (_, n) in enumerate(segments) for _ in range(n)], dtype=torch.int32)
    want_z, want_state = conv_reference(p, taps, b, state, segments)
    sd = dev(state)
    z = ops.shortconv(dev(p), dev(taps), None if b is None else dev(b), sd, dev(seg_start),
                      dev(seg_slot), dev(tok_seg), len(segments), torch.bfloat16)
    close(z, want_z, 2.0 ** -7, "conv output")
    close(sd, want_state, 1e-6, "conv state")
    # and the same bits as the per-token kernel that short batches take
    cut = 200
    sd2 = dev(state)
    parts = []
    for lo, hi in ((0, cut), (cut, T)):
        segs = []
        t = 0
        for slot, n in segments:
            a, e = max(t, lo), min(t + n, hi)
            if e > a:
                segs.append((slot, e - a))
            t += n
        ss = torch.tensor(np.cumsum([0] + [n for _, n in segs]), dtype=torch.int32)
        sl = torch.tensor([s_ for s_, _ in segs], dtype=torch.int32)
        ts = torch.tensor([i for i, (_, n) in enumerate(segs) for _ in range(n)], dtype=torch.int32)
        parts.append(ops.shortconv(dev(p[lo:hi]), dev(taps), None if b is None else dev(b), sd2,
                                   dev(ss), dev(sl), dev(ts), len(segs), torch.bfloat16))
    assert torch.equal(torch.cat(parts), z) and torch.equal(sd2, sd)


@pytest.mark.parametrize("n_requests,H,L,bias", [(300, 64, 3, True), (40, 72, 4, False), (257, 40, 2, True),
                                                 (300, 48, 5, False)])
def test_shortconv_of_hundreds_of_decoding_requests(n_requests, H, L, bias):
    """A decode step of a large batch: every segment one token, every one with a slot of its own, in
    an order that is not the slots' (all the work is at the segments' heads)."""
    from flyweight_b200.kernels import ops
    g = torch.Generator().manual_seed(n_requests + H)
    slots = torch.randperm(n_requests + 3, generator=g)[:n_requests].tolist()
    segments = [(slot, 1) for slot in slots]
    p = torch.randn(n_requests, 3 * H, generator=g).to(torch.bfloat16)
    taps = torch.randn(H, L, generator=g)
    b = torch.randn(H, generator=g) if bias else None
    state = torch.randn(n_requests + 3, H, L - 1, generator=g)
    seg_start = torch.arange(n_requests + 1, dtype=torch.int32)
    seg_slot = torch.tensor(slots, dtype=torch.int32)
    tok_seg = torch.arange(n_requests, dtype=torch.int32)
    want_z, want_state = conv_reference(p, taps, b, state, segments)
    sd = dev(state)
    z = ops.shortconv(dev(p), dev(taps), None if b is None else dev(b), sd, dev(seg_start),
                      dev(seg_slot), dev(tok_seg), n_requests, torch.bfloat16)
    close(z, want_z, 2.0 ** -7, "conv output")
    close(sd, want_state, 1e-6, "conv state")
    # the same step in two halves (fewer than 256 tokens each: the other kernel) gives the same bits
    sd2 = dev(state)
    half = n_requests // 2
    parts = []
    for lo, hi in ((0, half), (half, n_requests)):
        parts.append(ops.shortconv(dev(p[lo:hi]), dev(taps), None if b is None else dev(b), sd2,
                                   dev(torch.arange(hi - lo + 1, dtype=torch.int32)), dev(seg_slot[lo:hi]),
                                   dev(torch.arange(hi - lo, dtype=torch.int32)), hi - lo, torch.bfloat16))
    assert torch.equal(torch.cat(parts), z) and torch.equal(sd2, sd)


@pytest.mark.parametrize("T", [1, 2, 3])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_shortconv_of_one_two_and_three_tokens_stays_inside_its_buffers(T, dtype, guard_bands):
    """The smallest steps there are, as one segment and as T segments of one token, with the state
    (read and advanced in place) inside guard bands as well as the output."""
    from flyweight_b200.kernels import ops
    H, L = 72, 3
    g = torch.Generator().manual_seed(T)
    for segments in ([(1, T)], [(slot, 1) for slot in range(T)]):
        p = torch.randn(T, 3 * H, generator=g).to(dtype)
        taps = torch.randn(H, L, generator=g)
        state = torch.randn(3, H, L - 1, generator=g)
        seg_start = torch.tensor(np.cumsum([0] + [n for _, n in segments]), dtype=torch.int32)
        seg_slot = torch.tensor([s for s, _ in segments], dtype=torch.int32)
        tok_seg = torch.tensor([i for i, (_, n) in enumerate(segments) for _ in range(n)], dtype=torch.int32)
        want_z, want_state = conv_reference(p, taps, None, state, segments)
        sd = torch.empty(state.shape, dtype=torch.float32, device=DEV).copy_(state)      # guarded
        z = ops.shortconv(dev(p), dev(taps), None, sd, dev(seg_start), dev(seg_slot), dev(tok_seg),
                          len(segments), dtype)
        close(z, want_z, 1e-5 if dtype == torch.float32 else 2.0 ** -7, "conv output")
        close(sd, want_state, 1e-6, "conv state")
        guard_bands.check()


def test_the_guard_bands_notice_a_write_past_an_output(guard_bands):
    out = torch.empty((5, 7), dtype=torch.float32, device=DEV)
    assert torch.isnan(out).all()                           # unwritten elements read as NaN
    out.zero_()
    guard_bands.check()
    out.as_strided((36,), (1,)).fill_(1.0)                  # one element past the end
    with pytest.raises(AssertionError, match="past its end"):
        guard_bands.check()
    guard_bands.forget()
    out = torch.empty(16, dtype=torch.int32, device=DEV)
    out.as_strided((4,), (1,), out.storage_offset() - 4).fill_(3)    # four elements before the start
    with pytest.raises(AssertionError, match="before its output"):
        guard_bands.check()
    guard_bands.forget()


def test_shortconv_cut_anywhere_gives_the_same_bits():
    from flyweight_b200.kernels import ops
    g = torch.Generator().manual_seed(3)
    H, L, T = 72, 4, 50
    p = torch.randn(T, 3 * H, generator=g)
    taps = torch.randn(H, L, generator=g)

    def run(cuts):
        state = torch.zeros(2, H, L - 1, device=DEV)
        outs = []
        pos = 0
        for n in cuts:
            outs.append(ops.shortconv(
                dev(p[pos:pos + n]), dev(taps), None, state,
                dev(torch.tensor([0, n], dtype=torch.int32)), dev(torch.tensor([1], dtype=torch.int32)),
                dev(torch.zeros(n, dtype=torch.int32)), 1, torch.float32))
            pos += n
        return torch.cat(outs), state

    whole, s0 = run([T])
    for cuts in ([1] * T, [2, 1, 3, 44], [49, 1], [3, 3, 3, 41]):
        got, s1 = run(cuts)
        assert torch.equal(got, whole) and torch.equal(s0, s1), cuts


# ------------------------------------------------------------------ q/k norm, rope, cache write
def rope_table(theta, rot, n):
    inv = theta ** (-torch.arange(rot // 2, dtype=torch.float64) * 2 / rot)
    ang = torch.arange(n, dtype=torch.float64)[:, None] * inv[None]
    return torch.stack([ang.cos(), ang.sin()], -1).float()


@pytest.mark.parametrize("nh,nkv,hd,rot", [(4, 2, 16, 16), (3, 1, 32, 32), (5, 5, 48, 32), (2, 1, 80, 80),
                                           (8, 2, 128, 64), (2, 2, 256, 256)])
@pytest.mark.parametrize("dtype,bf16_input", [(torch.float32, False), (torch.bfloat16, False),
                                              (torch.bfloat16, True)])
@pytest.mark.parametrize("pairing", ["half_split", "interleaved"])
def test_qk_norm_rope_and_cache_write(nh, nkv, hd, rot, dtype, bf16_input, pairing):
    from flyweight_b200.kernels import ops
    g = torch.Generator().manual_seed(nh * hd)
    T, pages, P_ = 6, 5, 64
    positions = torch.tensor([0, 1, 63, 64, 65, 130], dtype=torch.int32)
    tok_seg = torch.tensor([0, 0, 1, 1, 1, 0], dtype=torch.int32)
    table_rows = torch.tensor([[3, 1, 4], [0, 2, -1]], dtype=torch.int32)
    qkv = torch.randn(T, (nh + 2 * nkv) * hd, generator=g)
    if bf16_input:                                            # the engine's bfloat16 path: 16-byte lanes
        qkv = qkv.to(torch.bfloat16)
    wq, wk = 1 + 0.1 * torch.randn(hd, generator=g), 1 + 0.1 * torch.randn(hd, generator=g)
    eps, theta = 1e-5, 1e4
    table = rope_table(theta, rot, 200)
    k_pool = torch.full((pages, nkv, P_, hd), 7.0).to(dtype)
    v_pool = torch.full((pages, nkv, P_, hd), 7.0).to(dtype)
    kd, vd = dev(k_pool), dev(v_pool)
    q = ops.qk_norm_rope(dev(qkv), dev(wq), dev(wk), dev(table), dev(positions), dev(tok_seg),
                         dev(table_rows), kd, vd, nh, nkv, hd, rot, eps, dtype, pairing=pairing)

    def norm_rope(x, w, pos):                                 # x: [heads, hd] float64
        x = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * w.double()
        cs = table[pos].double()
        out = x.clone()
        if pairing == "interleaved":                          # pair i = channels (2i, 2i + 1)
            a, b = x[:, 0:rot:2], x[:, 1:rot:2]
            out[:, 0:rot:2] = a * cs[:, 0] - b * cs[:, 1]
            out[:, 1:rot:2] = b * cs[:, 0] + a * cs[:, 1]
            return out
        a, b = x[:, :rot // 2], x[:, rot // 2:rot]            # pair i = channels (i, i + rot/2)
        out[:, :rot // 2] = a * cs[:, 0] - b * cs[:, 1]
        out[:, rot // 2:rot] = b * cs[:, 0] + a * cs[:, 1]
        return out

    tol = 1e-5 if dtype == torch.float32 else 2.0 ** -7
    want_k, want_v = k_pool.double().clone(), v_pool.double().clone()
    for t in range(T):
        pos = int(positions[t])
        row = qkv[t].double()
        qh = row[:nh * hd].reshape(nh, hd)
        kh = row[nh * hd:(nh + nkv) * hd].reshape(nkv, hd)
        vh = row[(nh + nkv) * hd:].reshape(nkv, hd)
        close(q[t].reshape(nh, hd), norm_rope(qh, wq, pos), tol, f"q token {t}")
        page = int(table_rows[int(tok_seg[t]), pos // P_])
        want_k[page, :, pos % P_] = norm_rope(kh, wk, pos)
        want_v[page, :, pos % P_] = vh
    close(kd, want_k, tol, "k pool")                          # also: nothing else was written
    close(vd, want_v, tol, "v pool")


# ------------------------------------------------------------------ attention
def attention_reference(q, k_seq, v_seq, pos, window, scale, group):
    """One query token (heads x hd) over its sequence's keys [0..pos] (float64)."""
    nh = q.shape[0]
    lo = max(0, pos - window + 1) if window > 0 else 0
    out = torch.zeros_like(q)
    for h in range(nh):
        kv = h // group
        s = (k_seq[lo:pos + 1, kv] @ q[h]) * scale
        p = torch.softmax(s, 0)
        out[h] = p @ v_seq[lo:pos + 1, kv]
    return out


def build_paged(k_seqs, v_seqs, n_pages, dtype, shuffle_seed=0, fill=float("nan")):
    """Scatter per-sequence K/V ([len][nkv][hd]) into pools through a shuffled block table;
    everything that holds no token is filled with ``fill`` so that a read past a sequence's
    end poisons the result."""
    nkv, hd = k_seqs[0].shape[1:]
    order = torch.randperm(n_pages, generator=torch.Generator().manual_seed(shuffle_seed)).tolist()
    k_pool = torch.full((n_pages, nkv, 64, hd), fill, dtype=torch.float64)
    v_pool = torch.full((n_pages, nkv, 64, hd), fill, dtype=torch.float64)
    width = max(-(-k.shape[0] // 64) for k in k_seqs)
    table = torch.full((len(k_seqs), width), -1, dtype=torch.int32)
    for s, (k, v) in enumerate(zip(k_seqs, v_seqs)):
        for logical in range(-(-k.shape[0] // 64)):
            page = order.pop()
            table[s, logical] = page
            n = min(64, k.shape[0] - logical * 64)
            k_pool[page, :, :n] = k[logical * 64:logical * 64 + n].transpose(0, 1)
            v_pool[page, :, :n] = v[logical * 64:logical * 64 + n].transpose(0, 1)
    return k_pool.to(dtype), v_pool.to(dtype), table


def make_ctx(lens, new, table, k_pool, v_pool):
    """A step context over hand-made pools: segment s has lens[s] tokens cached after the step,
    the last new[s] of them brought by it."""
    from flyweight_b200.engine import Segment, StepBatch, StepContext
    segments = [Segment(f"s{i}", i, n - m, [0] * m, []) for i, (n, m) in enumerate(zip(lens, new))]
    batch = StepBatch(segments, [table.tolist()], DEV)
    cache = type("Cache", (), {})()
    cache.k_pool, cache.v_pool = dev(k_pool), dev(v_pool)
    return StepContext(batch, None, DEV), cache, batch.block_tables[0]


ATTN_SHAPES = [(4, 2, 16), (3, 1, 32), (6, 6, 48), (8, 1, 64), (32, 8, 64), (5, 5, 80), (16, 1, 128),
               (2, 1, 256)]


@pytest.mark.parametrize("nh,nkv,hd", ATTN_SHAPES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [0, 70])
def test_paged_attention_mixed_batch(nh, nkv, hd, dtype, window):
    """A prompt portion with a cached prefix, a whole short prompt and two decode tokens in one
    launch, over shuffled pages; rows past each sequence's end hold NaN."""
    from flyweight_b200.kernels import ops, attention as attention_kernels
    g = torch.Generator().manual_seed(nh + hd)
    lens = [200, 37, 129, 64]                 # tokens in the cache after this step
    new = [90, 37, 1, 1]                      # of which this step brings the last ...
    k_seqs = [bf16_round(torch.randn(n, nkv, hd, generator=g).double()) for n in lens]
    v_seqs = [bf16_round(torch.randn(n, nkv, hd, generator=g).double()) for n in lens]
    k_pool, v_pool, table = build_paged(k_seqs, v_seqs, 12, dtype, shuffle_seed=hd)
    qs, positions, tok_seg = [], [], []
    for s, (n, m) in enumerate(zip(lens, new)):
        for pos in range(n - m, n):
            qs.append(bf16_round(torch.randn(nh, hd, generator=g).double()))
            positions.append(pos)
            tok_seg.append(s)
    q = torch.stack(qs)
    scale = 1.0 / math.sqrt(hd)
    want = torch.stack([attention_reference(q[t], k_seqs[tok_seg[t]], v_seqs[tok_seg[t]], positions[t],
                                            window, scale, nh // nkv) for t in range(len(qs))])

    ctx, cache, table_dev = make_ctx(lens, new, table, k_pool, v_pool)
    qd = dev(q.reshape(len(qs), nh * hd).to(dtype))
    tol = 1e-5 if dtype == torch.float32 else 2.0 ** -7
    got = ops.attention_simt(qd, cache.k_pool, cache.v_pool, ctx.batch.positions, ctx.batch.tok_seg,
                             table_dev, nh, window, scale, dtype)
    close(got.reshape(-1, nh, hd), want, tol, "SIMT attention")
    got = attention_kernels.paged_attention(ctx, qd, cache, table_dev, nh, window, scale, dtype)
    close(got.reshape(-1, nh, hd), want, tol, "dispatched attention")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_a_far_key_among_hundreds_and_the_edges_of_pages(dtype):
    """Random keys hide a fault at one position; here one key per case is made to match the
    query so strongly that the output must be (almost) that key's value: a far key (position 3
    of 700), the last key of a page (63), the first of the next (64), and the query's own."""
    from flyweight_b200.kernels import ops
    g = torch.Generator().manual_seed(9)
    nh, nkv, hd, n = 4, 2, 64, 700
    scale = 1.0 / math.sqrt(hd)
    for target in (3, 63, 64, 639, 640, 699):
        k = bf16_round(torch.randn(n, nkv, hd, generator=g).double() * 0.1)
        v = bf16_round(torch.randn(n, nkv, hd, generator=g).double())
        direction = torch.zeros(hd, dtype=torch.float64)
        direction[target % hd] = 1.0
        k[target, :, :] = direction * 16.0
        q = (direction * 16.0).repeat(nh, 1)                  # score 256/8 = 32 above the rest
        k_pool, v_pool, table = build_paged([k], [v], 12, dtype, shuffle_seed=target)
        got = ops.attention_simt(dev(q.reshape(1, -1).to(dtype)), dev(k_pool), dev(v_pool),
                                 dev(torch.tensor([n - 1], dtype=torch.int32)),
                                 dev(torch.zeros(1, dtype=torch.int32)), dev(table), nh, 0, scale, dtype)
        want = attention_reference(q, k, v, n - 1, 0, scale, nh // nkv)
        close(got.reshape(nh, hd), want, 1e-5 if dtype == torch.float32 else 2.0 ** -7, f"target {target}")
        close(got.reshape(nh, hd)[0], v[target, 0], 1e-3 if dtype == torch.float32 else 2.0 ** -6,
              f"value of key {target}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_the_edge_of_a_window(dtype):
    """The key just outside the window shouts, the key just inside whispers: a kernel that is
    off by one at the window's edge returns the wrong value."""
    from flyweight_b200.kernels import ops
    g = torch.Generator().manual_seed(4)
    nh, nkv, hd, n, window = 2, 1, 32, 300, 100
    scale = 1.0 / math.sqrt(hd)
    pos = n - 1
    k = bf16_round(torch.randn(n, nkv, hd, generator=g).double() * 0.1)
    v = bf16_round(torch.randn(n, nkv, hd, generator=g).double())
    direction = torch.zeros(hd, dtype=torch.float64)
    direction[5] = 1.0
    k[pos - window, 0] = direction * 16.0                     # just outside: must be ignored
    k[pos - window + 1, 0] = direction * 8.0                  # just inside: must win
    q = (direction * 16.0).repeat(nh, 1)
    k_pool, v_pool, table = build_paged([k], [v], 6, dtype)
    got = ops.attention_simt(dev(q.reshape(1, -1).to(dtype)), dev(k_pool), dev(v_pool),
                             dev(torch.tensor([pos], dtype=torch.int32)), dev(torch.zeros(1, dtype=torch.int32)),
                             dev(table), nh, window, scale, dtype)
    want = attention_reference(q, k, v, pos, window, scale, nh)
    tol = 1e-5 if dtype == torch.float32 else 2.0 ** -7
    close(got.reshape(nh, hd), want, tol, "window edge")
    close(got.reshape(nh, hd)[0], v[pos - window + 1, 0], 1e-3 if dtype == torch.float32 else 2.0 ** -6,
          "the key just inside the window")


def test_kernels_refuse_what_they_cannot_take():
    from flyweight_b200.kernels import KernelError, ops
    q = torch.zeros(1, 17 * 16, device=DEV)
    pool = torch.zeros(2, 1, 64, 16, device=DEV)
    i32 = lambda *v: torch.tensor(v, dtype=torch.int32, device=DEV)
    with pytest.raises(KernelError, match="unsupported"):     # 17 query heads on one KV head
        ops.attention_simt(q, pool, pool, i32(0), i32(0), i32(0).reshape(1, 1), 17, 0, 1.0, torch.float32)
    with pytest.raises(KernelError, match="unsupported"):     # 17 taps
        ops.shortconv(torch.zeros(1, 12, device=DEV), torch.zeros(4, 17, device=DEV), None,
                      torch.zeros(1, 4, 16, device=DEV), i32(0, 1), i32(0), i32(0), 1, torch.float32)
    with pytest.raises(KernelError, match="contiguous"):
        ops.gemm_simt(torch.zeros(4, 8, device=DEV).t(), torch.zeros(3, 4, device=DEV), torch.float32)


# ------------------------------------------------------------------ sampling
@pytest.mark.parametrize("rows", [5, 70])            # few rows: cut into slices; many: one block a row
@pytest.mark.parametrize("V", [100, 384, 65536, 50001])
def test_argmax_takes_the_lowest_id_among_equals(V, rows):
    from flyweight_b200.sampling import sampler
    g = torch.Generator().manual_seed(V)
    logits = torch.randn(rows, V, generator=g)
    logits[1, [7, V - 1]] = 50.0
    logits[2, :] = 0.0
    logits[3, V - 1] = 99.0
    want = [int(np.lexsort((np.arange(V), -row.numpy()))[0]) for row in logits]
    assert sampler.argmax(dev(logits)).tolist() == want
    assert want[1] == 7 and want[2] == 0 and want[3] == V - 1


@pytest.mark.parametrize("V", [384, 4099, 5000, 65536])      # 4099: rows that do not start on 16 bytes
def test_sampling_equals_the_plain_sampler_draw_for_draw(V):
    from flyweight_b200.sampling import SamplingConfig, sampler
    g = torch.Generator().manual_seed(V + 1)
    settings = [dict(temperature=0.8, top_k=40, top_p=0.95, min_p=0.05),
                dict(temperature=1.5, top_k=5, top_p=1.0, min_p=0.0),
                dict(temperature=0.3, top_k=1000, top_p=0.5, min_p=0.0),
                dict(temperature=1.0, top_k=0, top_p=0.9, min_p=0.01),
                dict(temperature=0.0, top_k=20, top_p=0.95, min_p=0.0),
                dict(temperature=2.0, top_k=1, top_p=1.0, min_p=0.0),
                dict(temperature=1.0, top_k=300, top_p=1.0, min_p=0.5),
                dict(temperature=1.2, top_k=3000, top_p=0.8, min_p=0.0),     # more candidates than are ever sorted
                dict(temperature=0.7, top_k=0, top_p=1.0, min_p=0.0)]        # the whole vocabulary, no cut at all
    for trial in range(6):
        logits = torch.randn(len(settings), V, generator=g) * 3
        logits[:, 11] = logits[:, 13]                          # ties inside the candidates
        rngs = [P.XorShift64Star(100 + trial * 10 + i) for i in range(len(settings))]
        uniforms = [P.XorShift64Star(100 + trial * 10 + i).uniform() for i in range(len(settings))]
        want = [P.sample(logits[i].numpy(), rng=rngs[i], **s) for i, s in enumerate(settings)]
        got = sampler.sample(dev(logits), [SamplingConfig(**s) for s in settings], uniforms).tolist()
        assert got == want, (trial, got, want)


@pytest.mark.parametrize("rows,V", [(3, 4099), (40, 5000), (150, 1000), (300, 65536)])
def test_sampling_with_fewer_ctas_a_row_draws_the_same_tokens(rows, V):
    """Eight CTAs share a row when there are few rows, four, two or one as rows fill the GPU by
    themselves; the masses are integers, so every cut of a row gives the same sums and the same draw."""
    from flyweight_b200.sampling import SamplingConfig, sampler
    g = torch.Generator().manual_seed(rows + V)
    kinds = [dict(temperature=0.8, top_k=40, top_p=0.95, min_p=0.05), dict(temperature=1.0, top_k=0, top_p=0.9, min_p=0.01),
             dict(temperature=1.2, top_k=3000, top_p=0.8, min_p=0.0), dict(temperature=0.0, top_k=20, top_p=0.95, min_p=0.0),
             dict(temperature=0.7, top_k=20, top_p=1.0, min_p=0.0, repetition_penalty=1.3)]
    settings = [kinds[i % len(kinds)] for i in range(rows)]
    logits = dev(torch.randn(rows, V, generator=g) * 3)
    uniforms = [P.XorShift64Star(7 + i).uniform() for i in range(rows)]
    recents = [[int(t) for t in torch.randint(0, V, (9,), generator=g)] for _ in range(rows)]
    configs = [SamplingConfig(**s) for s in settings]
    drawn = {}
    try:
        for ctas in (0, 8, 4, 2, 1):
            sampler.set_ctas_per_row(ctas)
            drawn[ctas] = sampler.sample(logits, configs, uniforms, recents).tolist()
    finally:
        sampler.set_ctas_per_row(0)
    for ctas in (8, 4, 2, 1):
        assert drawn[ctas] == drawn[0], f"{ctas} CTAs a row"
    for i in range(min(rows, 12)):                        # and they are the plain sampler's
        if "repetition_penalty" not in settings[i]:
            want = P.sample(logits[i].cpu().numpy(), rng=P.XorShift64Star(7 + i), **settings[i])
            assert drawn[0][i] == want, i


def test_sampling_rows_that_defeat_the_shortlist():
    """Rows on which the top-k search cannot narrow its bucket early, or narrows it to nothing: all
    logits equal, two values, thousands tied at the top, mostly -inf, one dominant value, a nearly flat
    row, a huge range, all negative.  The kernel falls back to walking the row; draws as the plain sampler's."""
    from flyweight_b200.sampling import SamplingConfig, sampler
    V = 20000
    g = torch.Generator().manual_seed(3)
    rows = [torch.zeros(V)]
    r = torch.zeros(V); r[::2] = 1.0; rows.append(r)
    rows.append(torch.randn(V, generator=g) * 30)
    r = torch.randn(V, generator=g); r[:18000] = -float("inf"); rows.append(r)
    r = torch.full((V,), -1e30); r[5] = 0.0; r[9] = -1.0; rows.append(r)
    rows.append(torch.randn(V, generator=g) * 1e-3)
    r = torch.randn(V, generator=g); r[100:3000] = 7.25; rows.append(r)
    rows.append(-torch.rand(V, generator=g) * 5 - 100)
    logits = torch.stack(rows)
    try:
        for settings in (dict(temperature=0.8, top_k=20, top_p=0.95, min_p=0.0),
                         dict(temperature=1.0, top_k=1000, top_p=0.9, min_p=0.01),
                         dict(temperature=0.7, top_k=0, top_p=0.9, min_p=0.0)):
            for ctas in (0, 1):
                sampler.set_ctas_per_row(ctas)
                for trial in range(2):
                    uniforms = [P.XorShift64Star(50 + trial * 20 + i).uniform() for i in range(len(rows))]
                    got = sampler.sample(dev(logits), [SamplingConfig(**settings)] * len(rows), uniforms).tolist()
                    want = [P.sample(logits[i].numpy(), rng=P.XorShift64Star(50 + trial * 20 + i), **settings)
                            for i in range(len(rows))]
                    assert got == want, (settings, ctas, trial)
    finally:
        sampler.set_ctas_per_row(0)


@pytest.mark.parametrize("V", [65536, 50001, 3000])     # 50001: odd rows do not start on 16 bytes (no estimate)
def test_sampling_whole_vocabulary_rows_from_flat_to_peaked(V):
    """A row that keeps more than 1,024 candidates looks for its top-p prefix among its 1,024 largest
    first, unless an estimate says it cannot be there: flat rows (the prefix is most of the row), rows at
    the edge (a prefix of about 1,024) and peaked rows (a handful) all draw the plain sampler's token."""
    from flyweight_b200.sampling import SamplingConfig, sampler
    g = torch.Generator().manual_seed(V + 5)
    spreads = [0.01, 0.5, 1.0, 2.0, 2.6, 2.8, 3.0, 3.2, 3.5, 4.0, 6.0, 12.0]
    logits = torch.stack([torch.randn(V, generator=g) * s for s in spreads])
    for settings in (dict(temperature=0.8, top_k=0, top_p=0.95, min_p=0.0),
                     dict(temperature=1.0, top_k=0, top_p=0.5, min_p=0.02),
                     dict(temperature=0.6, top_k=2000, top_p=0.99, min_p=0.0)):
        for trial in range(3):
            uniforms = [P.XorShift64Star(900 + trial * 20 + i).uniform() for i in range(len(spreads))]
            got = sampler.sample(dev(logits), [SamplingConfig(**settings)] * len(spreads), uniforms).tolist()
            want = [P.sample(logits[i].numpy(), rng=P.XorShift64Star(900 + trial * 20 + i), **settings)
                    for i in range(len(spreads))]
            assert got == want, (settings, trial)


def test_penalties_act_on_the_candidates():
    from flyweight_b200.sampling import SamplingConfig, sampler
    logits = torch.zeros(2, 50)
    logits[:, 4], logits[:, 9], logits[:, 2] = 5.0, 4.5, 4.0
    greedy = SamplingConfig(temperature=0.0, top_k=20, top_p=1.0, min_p=0.0, repetition_penalty=1.5)
    got = sampler.sample(dev(logits), [greedy, greedy], [0.0, 0.0], [[4, 4, 7], []]).tolist()
    assert got == [9, 4]              # 5.0/1.5 < 4.5: the repeated token loses; no history: it wins
    freq = SamplingConfig(temperature=0.0, top_k=20, top_p=1.0, min_p=0.0, frequency_penalty=0.3,
                          presence_penalty=0.2)
    got = sampler.sample(dev(logits), [freq, freq], [0.0, 0.0], [[4], [4, 4, 9, 9, 9]]).tolist()
    assert got == [4, 4]              # 5-0.5=4.5 ties 4.5 -> lower id; 5-0.8=4.2 > 4.5-1.1


def test_penalties_over_the_whole_vocabulary_and_above_1024_candidates():
    """Rows that keep more than 1,024 candidates are never sorted; their penalties act on the row
    itself before the cut (src/flyweight/v2.py:1497-1518).  Against that rule in numpy followed by
    the plain sampler, draw for draw, beside rows of the sorted path in the same launch."""
    from collections import Counter
    from flyweight_b200.sampling import SamplingConfig, sampler
    V = 5000
    g = torch.Generator().manual_seed(77)
    settings = [dict(temperature=0.9, top_k=0, top_p=0.9, min_p=0.0, repetition_penalty=1.7,
                     presence_penalty=0.5, frequency_penalty=0.25),
                dict(temperature=0.0, top_k=0, top_p=1.0, min_p=0.0, repetition_penalty=2.0),
                dict(temperature=1.1, top_k=3000, top_p=1.0, min_p=0.01, frequency_penalty=1.5, penalty_window=5),
                dict(temperature=0.8, top_k=40, top_p=0.95, min_p=0.05, repetition_penalty=1.3)]
    for trial in range(5):
        logits = torch.randn(len(settings), V, generator=g) * 3
        best = [int(i) for i in logits.argmax(dim=1)]
        recents = [[best[0], best[0], 17, best[0], 4999], [best[1], 3], [1, 2, best[2], best[2], best[2], best[2], 9],
                   [best[3], 11]]
        uniforms = [P.XorShift64Star(300 + trial * 10 + i).uniform() for i in range(len(settings))]
        want = []
        for i, s in enumerate(settings):
            row = logits[i].numpy().copy()
            cfg = SamplingConfig(**s)
            if (s["top_k"] or V) > 1024:
                window = recents[i][-cfg.penalty_window:]
                for t, count in Counter(window).items():
                    value = row[t]
                    if cfg.repetition_penalty != 1.0:
                        value = value / np.float32(cfg.repetition_penalty) if value > 0 else value * np.float32(cfg.repetition_penalty)
                    value = np.float32(value) - np.float32(cfg.presence_penalty)
                    row[t] = np.float32(value) - np.float32(cfg.frequency_penalty) * np.float32(count)
                want.append(P.sample(row, rng=P.XorShift64Star(300 + trial * 10 + i), temperature=s["temperature"],
                                     top_k=s["top_k"], top_p=s["top_p"], min_p=s["min_p"]))
            else:
                want.append(None)
        device_logits = dev(logits)
        kept = device_logits.clone()
        got = sampler.sample(device_logits, [SamplingConfig(**s) for s in settings], uniforms, recents).tolist()
        assert torch.equal(device_logits, kept)                    # the caller's logits are not touched
        assert got[:3] == want[:3], (trial, got, want)
        assert got[1] != best[1]                                   # the repeated best token lost its place
        alone = sampler.sample(dev(logits[3:]), [SamplingConfig(**settings[3])], uniforms[3:], recents[3:]).tolist()
        assert got[3] == alone[0]                                  # the sorted path is as it was


# ------------------------------------------------------------------ tcgen05 matrix products
TC_SHAPES = [(1, 128, 64), (16, 128, 256), (8, 2048, 2048), (64, 6144, 2048), (100, 200, 96),
             (17, 100, 72), (300, 1000, 264), (129, 384, 96), (2048, 2048, 512), (8, 512, 8192)]


@pytest.mark.parametrize("M,N,K", TC_SHAPES)
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_tcgen05_gemm(M, N, K, out_dtype):
    from flyweight_b200.kernels import tensorcore as tc
    g = torch.Generator().manual_seed(M * 7 + N + K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    assert tc.accepts(dev(x), dev(w), out_dtype)
    want = x.double() @ w.double().T
    tol = 1e-5 if out_dtype == torch.float32 else 2.0 ** -8
    close(tc.gemm(dev(x), dev(w), out_dtype), want, tol, "tcgen05")
    assert tc.status() == 0


@pytest.mark.parametrize("splits", [1, 2, 3, 5, 8])
@pytest.mark.parametrize("M", [1, 16, 40, 64, 100, 128, 300])
def test_tcgen05_split_k_over_a_cluster(splits, M):
    from flyweight_b200.kernels import tensorcore as tc
    g = torch.Generator().manual_seed(splits * 100 + M)
    N, K = 384, 1096                                           # 17.1 k-blocks: ragged last split
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    add = torch.randn(M, N, generator=g)
    want = x.double() @ w.double().T
    tile = 128 if M > 64 else 0                      # more than 64 tokens: 128-token tiles
    first = tc.gemm(dev(x), dev(w), torch.float32, None, splits, 0, tile)
    close(first, want, 1e-5, f"split {splits}")
    assert torch.equal(first, tc.gemm(dev(x), dev(w), torch.float32, None, splits, 0, tile))   # deterministic
    close(tc.gemm(dev(x), dev(w), torch.float32, dev(add), splits, 0, tile), want + add.double(), 1e-5, "addend")
    assert tc.status() == 0


@pytest.mark.parametrize("M,F,K", [(1, 128, 64), (8, 8192 // 8, 2048), (40, 192, 64), (64, 320, 96),
                                   (200, 320, 96), (700, 1000, 264)])
def test_tcgen05_swiglu_epilogue(M, F, K):
    from flyweight_b200.kernels import tensorcore as tc
    g = torch.Generator().manual_seed(M + F)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(2 * F, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    gu = x.double() @ w.double().T
    want = torch.from_numpy(P.silu(gu[:, :F].numpy())) * gu[:, F:]
    close(tc.swiglu_gate_up(dev(x), dev(w)), want, 2.0 ** -8, "swiglu")
    assert tc.status() == 0


@pytest.mark.parametrize("M,N,K", [(1, 128, 64), (8, 384, 2048), (16, 200, 96), (17, 256, 512), (40, 320, 264),
                                   (64, 2048, 1024)])
@pytest.mark.parametrize("splits", [1, 2, 4, 8])
def test_tcgen05_gemm_with_the_norm_folded_in(M, N, K, splits):
    """rmsnorm(x) @ W^T in one kernel: the kernel builds its activation tiles from the fp32
    residual, sums the squares per slice of K and scales the accumulator at the end."""
    from flyweight_b200.kernels import tensorcore
    g = torch.Generator().manual_seed(M + N + K + splits)
    x = torch.randn(M + 3, K, generator=g) * torch.linspace(0.1, 30.0, M + 3)[:, None]   # rows of very different size
    nw = 1 + 0.2 * torch.randn(K, generator=g)
    w = bf16_round(torch.randn(N, K, generator=g) / math.sqrt(K))
    eps = 1e-5
    rows = torch.randperm(M + 3, generator=g)[:M].to(torch.int32)
    for use_rows in (False, True):
        src = x[rows.long()] if use_rows else x[:M]
        normed = src.double() * torch.rsqrt((src.double() ** 2).mean(-1, keepdim=True) + eps) * nw.double()
        want = normed @ w.double().T
        xin = dev(x) if use_rows else dev(x[:M].contiguous())
        for out_dtype in (torch.float32, torch.bfloat16):
            got = tensorcore.gemm_normed(xin, dev(nw), eps, dev(w, torch.bfloat16), out_dtype,
                                         rows=dev(rows) if use_rows else None, splits=splits)
            assert tensorcore.status() == 0
            close(got, want, 2.0 ** -7, f"normed gemm rows={use_rows} {out_dtype}")


@pytest.mark.parametrize("M,F,K", [(1, 128, 64), (8, 1024, 2048), (40, 192, 128), (64, 320, 96)])
def test_tcgen05_swiglu_with_the_norm_folded_in(M, F, K):
    from flyweight_b200.kernels import tensorcore
    g = torch.Generator().manual_seed(M + F + K)
    x = torch.randn(M, K, generator=g) * 3.0
    nw = 1 + 0.2 * torch.randn(K, generator=g)
    w = bf16_round(torch.randn(2 * F, K, generator=g) / math.sqrt(K))
    eps = 1e-6
    normed = x.double() * torch.rsqrt((x.double() ** 2).mean(-1, keepdim=True) + eps) * nw.double()
    gate, up = normed @ w[:F].double().T, normed @ w[F:].double().T
    want = gate * torch.sigmoid(gate) * up
    for splits in (1, 2, 4):
        got = tensorcore.swiglu_gate_up_normed(dev(x), dev(nw), eps, dev(w, torch.bfloat16), splits=splits)
        assert tensorcore.status() == 0
        close(got, want, 2.0 ** -6, f"normed swiglu splits={splits}")


def test_a_wait_that_runs_out_is_reported_and_the_device_stays_usable():
    """Every wait in the tensor-core kernels is bounded.  A one-thread kernel waits on a barrier
    that nothing arrives on; it must give up, leave its code in the status word that the
    runner's health check raises on, and the next product must run as usual."""
    from flyweight_b200.kernels import KernelError, lib, tensorcore
    from flyweight_b200.kernels.lib import stream
    assert tensorcore.status() == 0
    lib.call("fwb_selftest_bounded_wait", 77, stream())
    torch.cuda.synchronize()
    assert tensorcore.status() == 77
    assert tensorcore.status() == 0                          # reading clears it
    lib.call("fwb_selftest_bounded_wait", 78, stream())
    checker = type("R", (), {})()
    checker.bad_token_flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    from flyweight_b200.engine.runner import ModelRunner
    with pytest.raises(KernelError, match="gave up"):
        ModelRunner.check_health(checker)
    g = torch.Generator().manual_seed(1)
    x, w = torch.randn(8, 256, generator=g).to(torch.bfloat16), torch.randn(128, 256, generator=g).to(torch.bfloat16)
    close(tensorcore.gemm(dev(x), dev(w), torch.float32), x.double() @ w.double().T, 1e-5, "after the self-test")
    assert tensorcore.status() == 0


def test_tcgen05_swiglu_in_two_launches_cut_at_a_whole_wave():
    """2,048 tokens x 8,192 features make 3.46 waves of CTAs: the product runs as 55 feature tiles
    with 256-token tiles and 9 with 128-token tiles.  Same bits as one launch, right against fp64."""
    from flyweight_b200.kernels import tensorcore
    _swiglu_two_launches(2048, 8192, 64)
    _swiglu_two_launches(2000, 8100, 72)         # ragged tokens and features on both sides of the cut


def _swiglu_two_launches(M, F, K):
    from flyweight_b200.kernels import tensorcore
    assert tensorcore._wave_cut(M, F) == 55
    g = torch.Generator().manual_seed(2)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(2 * F, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    two = tensorcore.swiglu_gate_up(dev(x), dev(w))
    one = tensorcore.swiglu_gate_up(dev(x), dev(w), tile_tokens=256)
    assert tensorcore.status() == 0
    assert torch.equal(two, one)
    gate, up = x.double() @ w[:F].double().T, x.double() @ w[F:].double().T
    close(two, gate * torch.sigmoid(gate) * up, 2.0 ** -6, "swiglu in two launches")


def test_tcgen05_pair_gemm_in_two_launches_cut_at_a_whole_round():
    """2,048 tokens x 6,144 features are 96 wide pairs, 1.3 rounds of 74: nine 512-feature blocks
    run wide, the last three as one-block pairs.  Same bits as the one-launch forms."""
    from flyweight_b200.kernels import tensorcore
    M, N, K = 2048, 6144, 128
    assert tensorcore._pair_wave_cut(M, N) == 9
    g = torch.Generator().manual_seed(6)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    for out_dtype in (torch.bfloat16, torch.float32):
        two = tensorcore.gemm_pair(dev(x), dev(w), out_dtype, wide=True)
        narrow = tensorcore.gemm_pair(dev(x), dev(w), out_dtype, wide=False)
        assert tensorcore.status() == 0
        assert torch.equal(two, narrow)
        close(two, x.double() @ w.double().T, 1e-5 if out_dtype == torch.float32 else 2.0 ** -8, "pair gemm in two launches")


def test_tcgen05_refuses_what_tma_cannot_address():
    from flyweight_b200.kernels import KernelError, tensorcore as tc
    x = torch.zeros(4, 100, dtype=torch.bfloat16, device=DEV)   # K not a multiple of 8
    w = torch.zeros(128, 100, dtype=torch.bfloat16, device=DEV)
    assert not tc.accepts(x, w, torch.float32)
    with pytest.raises(KernelError, match="unsupported"):
        tc.gemm(x, w, torch.float32)
    assert not tc.accepts(x.float(), w, torch.float32)


@pytest.mark.parametrize("nh,nkv,hd", [(4, 2, 16), (3, 1, 32), (32, 8, 64), (6, 2, 80), (16, 1, 128), (5, 5, 48)])
@pytest.mark.parametrize("window", [0, 100])
def test_decode_attention_over_split_contexts(nh, nkv, hd, window):
    """A step of single tokens at very different context lengths (1 .. 1500 keys): the
    tensor-core decode kernel with the context cut into slices, merged, against fp64."""
    from flyweight_b200.kernels import attention as attention_kernels, ops
    g = torch.Generator().manual_seed(nh * 3 + hd)
    lens = [1, 64, 65, 700, 1500, 257]
    new = [1] * len(lens)
    k_seqs = [bf16_round(torch.randn(n, nkv, hd, generator=g).double()) for n in lens]
    v_seqs = [bf16_round(torch.randn(n, nkv, hd, generator=g).double()) for n in lens]
    k_pool, v_pool, table = build_paged(k_seqs, v_seqs, 48, torch.bfloat16, shuffle_seed=hd + 1)
    q = torch.stack([bf16_round(torch.randn(nh, hd, generator=g).double()) for _ in lens])
    scale = 1.0 / math.sqrt(hd)
    want = torch.stack([attention_reference(q[t], k_seqs[t], v_seqs[t], lens[t] - 1, window, scale, nh // nkv)
                        for t in range(len(lens))])
    ctx, cache, table_dev = make_ctx(lens, new, table, k_pool, v_pool)
    qd = dev(q.reshape(len(lens), nh * hd).to(torch.bfloat16))
    assert ctx.batch.max_segment == 1
    got = attention_kernels.paged_attention(ctx, qd, cache, table_dev, nh, window, scale, torch.bfloat16)
    close(got.reshape(-1, nh, hd), want, 2.0 ** -7, "decode attention")
    for splits, per in ((1, 24), (2, 12), (5, 5), (24, 1)):
        got = ops.attention_decode_mma(qd, cache.k_pool, cache.v_pool, ctx.batch.positions, ctx.batch.tok_seg,
                                       table_dev, nh, window, scale, splits, per)
        close(got.reshape(-1, nh, hd), want, 2.0 ** -7, f"{splits} splits")
    for splits, per in ((2, 12), (3, 8), (5, 5), (8, 3)):        # the slices as a cluster, merged in the kernel
        got = ops.attention_decode_mma(qd, cache.k_pool, cache.v_pool, ctx.batch.positions, ctx.batch.tok_seg,
                                       table_dev, nh, window, scale, splits, per, merge_in_cluster=True)
        close(got.reshape(-1, nh, hd), want, 2.0 ** -7, f"{splits} splits in a cluster")
    if hd in (64, 128):
        # at these head sizes the tiles come by TMA (swizzled boxes, an mbarrier a stage); by cp.async
        # into padded rows the same numbers go through the same arithmetic: the same bits
        for splits, per, cluster in ((1, 24, False), (5, 5, False), (24, 1, False), (3, 8, True), (8, 3, True)):
            run = lambda: ops.attention_decode_mma(qd, cache.k_pool, cache.v_pool, ctx.batch.positions,
                                                   ctx.batch.tok_seg, table_dev, nh, window, scale, splits, per,
                                                   merge_in_cluster=cluster)
            by_tma = run()
            try:
                ops.set_decode_attention_tma(False)
                by_cp_async = run()
            finally:
                ops.set_decode_attention_tma(True)
            assert torch.equal(by_tma, by_cp_async), (splits, per, cluster)
    from flyweight_b200.kernels import tensorcore
    assert tensorcore.status() == 0


@pytest.mark.parametrize("nh,nkv,hd,rot,pairing,normed,shares", [
    (32, 8, 64, 64, "half_split", True, False), (16, 1, 128, 64, "interleaved", True, False),
    (6, 2, 80, 32, "half_split", False, False), (4, 2, 16, 16, "half_split", True, False),
    (12, 4, 64, 0, "half_split", True, False), (8, 2, 64, 32, "interleaved", True, True)])
def test_decode_attention_that_norms_turns_and_stores_its_own_token(nh, nkv, hd, rot, pairing, normed, shares):
    """A step of single tokens: the decode attention kernel does the q/k head norm, the rotation and
    the page write of its own token itself.  Against the two kernels that every other step uses (the
    norm-and-rotate kernel, then the attention): the same output bits and the same pools, at page edges
    (positions 0, 63, 64), with the context in one piece, in slices, in a cluster; with partial and no
    rotation, both pairings, no norm, and a layer that reads another layer's cache and writes none."""
    from flyweight_b200.kernels import ops
    g = torch.Generator().manual_seed(nh * 5 + hd + rot)
    lens = [1, 64, 65, 700, 1500, 257, 128]
    n_kv_in = 0 if shares else nkv
    k_seqs = [bf16_round(torch.randn(n, nkv, hd, generator=g).double()) for n in lens]
    v_seqs = [bf16_round(torch.randn(n, nkv, hd, generator=g).double()) for n in lens]
    k_pool, v_pool, table = build_paged(k_seqs, v_seqs, 48, torch.bfloat16, shuffle_seed=hd + 2, fill=0.0)
    ctx, cache, table_dev = make_ctx(lens, [1] * len(lens), table, k_pool, v_pool)
    qkv = dev((torch.randn(len(lens), (nh + 2 * n_kv_in) * hd, generator=g) * 2).to(torch.bfloat16))
    q_norm = dev(torch.rand(hd, generator=g) + 0.5) if normed else None
    k_norm = dev(torch.rand(hd, generator=g) + 0.5) if normed else None
    half = max(1, rot // 2)
    angle = torch.arange(1600, dtype=torch.float64)[:, None] * torch.rand(half, generator=g).double()[None]
    rope = dev(torch.stack([angle.cos(), angle.sin()], -1).float().contiguous())
    scale = 1.0 / math.sqrt(hd)
    pos, seg = ctx.batch.positions, ctx.batch.tok_seg
    for splits, per, cluster in ((1, 24, False), (3, 8, True), (8, 3, True), (5, 5, False), (24, 1, False)):
        two = [cache.k_pool.clone(), cache.v_pool.clone()]
        q = ops.qk_norm_rope(qkv, q_norm, k_norm, rope, pos, seg, table_dev if n_kv_in else None,
                             two[0] if n_kv_in else None, two[1] if n_kv_in else None, nh, n_kv_in, hd, rot, 1e-5,
                             torch.bfloat16, pairing=pairing)
        want = ops.attention_decode_mma(q, two[0], two[1], pos, seg, table_dev, nh, 0, scale, splits, per,
                                        merge_in_cluster=cluster)
        one = [cache.k_pool.clone(), cache.v_pool.clone()]
        got = ops.attention_decode_fused(qkv, q_norm, k_norm, rope, rot, 1e-5, pairing, n_kv_in, one[0], one[1], pos,
                                         seg, table_dev, nh, 0, scale, splits, per, merge_in_cluster=cluster)
        assert torch.equal(got, want), (splits, per, cluster)
        assert torch.equal(one[0], two[0]) and torch.equal(one[1], two[1]), "pools"
        if n_kv_in:
            assert not torch.equal(one[0], cache.k_pool)         # the keys of this step were written
    from flyweight_b200.kernels import tensorcore
    assert tensorcore.status() == 0


def test_tensor_core_attention_finds_a_far_key_and_the_window_edge():
    from flyweight_b200.kernels import attention as attention_kernels
    g = torch.Generator().manual_seed(12)
    nh, nkv, hd, n = 4, 2, 64, 700
    scale = 1.0 / math.sqrt(hd)
    for target, window in ((3, 0), (63, 0), (64, 0), (639, 0), (640, 0), (699, 0), (600, 100), (599, 100)):
        k = bf16_round(torch.randn(n, nkv, hd, generator=g).double() * 0.1)
        v = bf16_round(torch.randn(n, nkv, hd, generator=g).double())
        direction = torch.zeros(hd, dtype=torch.float64)
        direction[target % hd] = 1.0
        k[target, :, :] = direction * 16.0
        q = (direction * 16.0).repeat(nh, 1)
        k_pool, v_pool, table = build_paged([k], [v], 12, torch.bfloat16, shuffle_seed=target)
        want = attention_reference(q, k, v, n - 1, window, scale, nh // nkv)
        for new in (1, 5, 100):                              # decode, tiled mma.sync and tcgen05 kernels
            ctx, cache, table_dev = make_ctx([n], [new], table, k_pool, v_pool)
            qd = dev(q.reshape(1, -1).to(torch.bfloat16).repeat(new, 1))
            got = attention_kernels.paged_attention(ctx, qd, cache, table_dev, nh, window, scale, torch.bfloat16)
            close(got[-1].reshape(nh, hd), want, 2.0 ** -7, f"target {target} window {window} new {new}")
            if window == 0 or target > n - 1 - window:
                close(got[-1].reshape(nh, hd)[0], v[target, 0], 2.0 ** -6, f"value of key {target}")
            else:                                            # the shouting key is outside the window
                assert (got[-1].reshape(nh, hd)[0].double().cpu() - v[target, 0]).abs().max() > 0.1


@pytest.mark.parametrize("nh,nkv,hd", [(32, 8, 64), (8, 1, 64), (3, 1, 64), (16, 2, 128), (2, 2, 128)])
@pytest.mark.parametrize("window", [0, 100])
def test_tcgen05_prompt_attention(nh, nkv, hd, window):
    """Prompt portions on the tcgen05 kernel: a whole prompt over several 128-row tiles, a
    portion behind a cached prefix that starts inside a page, a prompt that ends on a page's
    first key, a single token; shuffled pages, NaN wherever no key was written."""
    from flyweight_b200.kernels import ops
    g = torch.Generator().manual_seed(nh * hd + window)
    lens = [300, 200, 65, 129]
    new = [300, 130, 65, 1]
    k_seqs = [bf16_round(torch.randn(n, nkv, hd, generator=g).double()) for n in lens]
    v_seqs = [bf16_round(torch.randn(n, nkv, hd, generator=g).double()) for n in lens]
    k_pool, v_pool, table = build_paged(k_seqs, v_seqs, 16, torch.bfloat16, shuffle_seed=hd + nh)
    qs, positions, tok_seg = [], [], []
    for s_, (n, m) in enumerate(zip(lens, new)):
        for pos in range(n - m, n):
            qs.append(bf16_round(torch.randn(nh, hd, generator=g).double()))
            positions.append(pos)
            tok_seg.append(s_)
    q = torch.stack(qs)
    scale = 1.0 / math.sqrt(hd)
    want = torch.stack([attention_reference(q[t], k_seqs[tok_seg[t]], v_seqs[tok_seg[t]], positions[t],
                                            window, scale, nh // nkv) for t in range(len(qs))])
    ctx, cache, table_dev = make_ctx(lens, new, table, k_pool, v_pool)
    qd = dev(q.reshape(len(qs), nh * hd).to(torch.bfloat16))
    per_tile = max(1, 128 // (nh // nkv))
    tile_seg, tile_tok0, n_tiles = ctx.batch.attention_tiles(per_tile)
    got = ops.attention_prefill_tcgen05(qd, cache.k_pool, cache.v_pool, ctx.batch.positions,
                                        ctx.batch.seg_start, tile_seg, tile_tok0, n_tiles, per_tile,
                                        table_dev, nh, window, scale)
    from flyweight_b200.kernels import tensorcore
    assert tensorcore.status() == 0
    close(got.reshape(-1, nh, hd), want, 2.0 ** -7, "tcgen05 attention")


@pytest.mark.parametrize("M,N,K", [(600, 1000, 264), (300, 256, 64), (257, 3072, 512), (1030, 700, 96)])
@pytest.mark.parametrize("tile_tokens,wide", [(256, 1), (128, 1), (128, 0), (256, 0)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_tcgen05_tile_shapes_for_prompts(M, N, K, tile_tokens, wide, out_dtype):
    """Token tiles of 128 and 256 and the two-feature-tile ("wide") form, on ragged edges."""
    from flyweight_b200.kernels import tensorcore as tc
    g = torch.Generator().manual_seed(M + N + K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    want = x.double() @ w.double().T
    got = tc.gemm(dev(x), dev(w), out_dtype, None, None, 0, tile_tokens, wide)
    close(got, want, 1e-5 if out_dtype == torch.float32 else 2.0 ** -8, "tile shape")
    assert tc.status() == 0


@pytest.mark.parametrize("M,N,K", [(129, 256, 64), (256, 256, 256), (300, 700, 264), (1030, 1000, 96),
                                   (2048, 2048, 512), (513, 3072, 200)])
@pytest.mark.parametrize("wide", [False, True])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_tcgen05_cta_pair_gemm(M, N, K, wide, out_dtype):
    """The cta_group::2 kernel: 256 features x 256 tokens per CTA pair, ragged edges included."""
    from flyweight_b200.kernels import tensorcore as tc
    g = torch.Generator().manual_seed(M + 3 * N + K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    want = x.double() @ w.double().T
    close(tc.gemm_pair(dev(x), dev(w), out_dtype, wide), want,
          1e-5 if out_dtype == torch.float32 else 2.0 ** -8, "pair gemm")
    assert tc.status() == 0


@pytest.mark.parametrize("M,F,K", [(200, 320, 96), (700, 1000, 264), (2048, 512, 128)])
def test_tcgen05_cta_pair_swiglu(M, F, K):
    from flyweight_b200.kernels import tensorcore as tc
    g = torch.Generator().manual_seed(M + F)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(2 * F, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    gu = x.double() @ w.double().T
    want = torch.from_numpy(P.silu(gu[:, :F].numpy())) * gu[:, F:]
    close(tc.swiglu_gate_up_pair(dev(x), dev(w)), want, 2.0 ** -8, "pair swiglu")
    assert tc.status() == 0


@pytest.mark.parametrize("M,N,K", [(65, 2048, 8192), (128, 384, 4168), (300, 2048, 4096), (256, 2048, 8192),
                                   (700, 260, 4104), (200, 1000, 5000)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_tcgen05_mid_size_products_split_k_over_128_token_tiles(M, N, K, out_dtype):
    """A few hundred tokens against a narrow matrix: 64- or 128-token tiles on single CTAs with K
    cut across a cluster instead of a handful of CTA pairs, whichever the cost model of that range
    puts first; the same numbers as with it switched off."""
    from flyweight_b200.kernels import tensorcore as tc
    g = torch.Generator().manual_seed(M + N + K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    want = x.double() @ w.double().T
    # fp32 out: the tensor core's accumulator loses a little with every block of K it adds
    tol = 1e-5 * max(1.0, K / 2048) if out_dtype == torch.float32 else 2.0 ** -8
    assert tc.mid_size_choice(256, 2048, 8192, 1, True) == ("single", 128, 4)      # w2 of LFM2-1.2B
    assert tc.mid_size_choice(128, 2048, 2048, 1, False) == ("single", 128, 4)    # out_proj
    assert tc.mid_size_choice(512, 6144, 2048, 1, True)[0] == "pair"              # in_proj
    assert tc.mid_size_choice(256, 8192, 2048, 2, False) == ("single", 128, 1)    # gate|up
    got = tc.gemm(dev(x), dev(w), out_dtype)
    close(got, want, tol, "mid-size split")
    tc.set_mid_size_split(False)
    try:
        close(tc.gemm(dev(x), dev(w), out_dtype), want, tol, "mid-size, as before")
    finally:
        tc.set_mid_size_split(True)
    assert tc.status() == 0
