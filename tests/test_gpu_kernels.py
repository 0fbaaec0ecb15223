"""Each kernel alone against a plain PyTorch float32 reference of the same operation, at sizes
other than the engine's tiny models: widths and vocabularies that are no power of two, head sizes
in steps of 16, odd head counts."""

import math

import pytest
import torch

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [pytest.param(torch.float32, id="f32"), pytest.param(torch.bfloat16, id="bf16")]


def K():
    from llm_pipeline_b200.ops import kernels
    return kernels


def tol(dtype, f32=1e-5, bf16=2e-2):
    return f32 if dtype == torch.float32 else bf16


def rnd(*shape, dtype=torch.float32, seed=0, scale=1.0):
    gen = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=gen) * scale).to(dtype).to(DEV)


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding(dtype):
    table = rnd(1000, 200, dtype=dtype)
    ids = torch.tensor([0, 999, 5, 5, 731], dtype=torch.int32, device=DEV)
    out = torch.empty(5, 200, dtype=torch.float32, device=DEV)
    K().embedding(ids, table, out)
    assert torch.equal(out, table[ids.long()].float())


def test_rope_tables_match_the_reference_formula():
    positions = torch.tensor([0, 1, 17, 4095, 100000], dtype=torch.int32, device=DEV)
    for head_dim, theta in ((48, 10000.0), (128, 1000000.0)):
        exponent = torch.arange(0, head_dim, 2, dtype=torch.int64).float() / head_dim
        inv_freq = (1.0 / (theta ** exponent)).to(DEV)
        cos = torch.empty(5, head_dim // 2, device=DEV)
        sin = torch.empty_like(cos)
        K().rope_tables(positions, inv_freq, 1.0, cos, sin)
        want_cos, want_sin = plain.rope_cos_sin(positions.cpu(), head_dim, theta)
        assert torch.allclose(cos.cpu(), want_cos[:, :head_dim // 2], atol=2e-6)
        assert torch.allclose(sin.cpu(), want_sin[:, :head_dim // 2], atol=2e-6)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H", [1000, 4096, 4096 + 16, 5120, 8192, 8200, 1002, 16384, 16400])       # 4096, 8192, 16384: blocks of 1024 threads
def test_add_rmsnorm(dtype, H):
    residual = rnd(7, H, seed=1)
    delta = rnd(7, H, dtype=dtype, seed=2)
    bias = rnd(H, seed=3, scale=0.1)
    weight = (1 + 0.1 * rnd(H, seed=4)).to(dtype)
    x = residual + delta.float() + bias
    want = plain.rms_norm(x, weight.float(), 1e-5)
    res = residual.clone()
    out = torch.empty(7, H, dtype=dtype, device=DEV)
    K().add_rmsnorm(res, delta, weight, 1e-5, out, delta_bias=bias)
    assert torch.allclose(res, x, atol=1e-6)
    assert torch.allclose(out.float(), want, atol=tol(dtype, 2e-5, 4e-2), rtol=tol(dtype, 1e-5, 1e-2))
    # selected rows: the residual is left alone
    rows = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEV)
    res2 = residual.clone()
    out2 = torch.empty(3, H, dtype=dtype, device=DEV)
    K().add_rmsnorm(res2, delta, weight, 1e-5, out2, delta_bias=bias, rows=rows)
    assert torch.equal(res2, residual)
    assert torch.equal(out2, out[rows.long()])
    # no addend: plain norm of the residual
    out3 = torch.empty(7, H, dtype=dtype, device=DEV)
    K().add_rmsnorm(res2, None, weight, 1e-5, out3)
    assert torch.allclose(out3.float(), plain.rms_norm(residual, weight.float(), 1e-5), atol=tol(dtype, 2e-5, 4e-2))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,rot", [(5, 5, 48, 48), (8, 2, 128, 128), (3, 1, 80, 32)])
def test_qkv_post_norm_rotary_and_page_write(dtype, nq, nkv, d, rot):
    N, page_size, pages_n = 11, 4, 9
    qkv = rnd(N, (nq + 2 * nkv) * d, dtype=dtype, seed=5)
    bias = rnd((nq + 2 * nkv) * d, seed=6, scale=0.1)
    qw, kw = (1 + 0.1 * rnd(d, seed=7)), (1 + 0.1 * rnd(d, seed=8))
    positions = torch.tensor([3, 4, 5, 6, 7, 8, 0, 1, 2, 90, 91], dtype=torch.int32, device=DEV)
    exponent = torch.arange(0, rot, 2, dtype=torch.int64).float() / rot
    inv_freq = (1.0 / (10000.0 ** exponent)).to(DEV)
    cos = torch.empty(N, rot // 2, device=DEV)
    sin = torch.empty_like(cos)
    K().rope_tables(positions, inv_freq, 1.0, cos, sin)
    slots = torch.tensor([20, 21, 22, 23, 4, 5, 35, 34, 33, -1, 0], dtype=torch.int32, device=DEV)
    pages = torch.zeros(pages_n, 2, nkv, page_size, d, dtype=dtype, device=DEV)
    work = qkv.clone()
    K().qkv_post(work, nq, nkv, d, bias=bias, q_weight=qw, k_weight=kw, eps=1e-6, cos=cos, sin=sin, rotary_dim=rot,
                 slots=slots, pages=pages, page_size=page_size)
    x = qkv.float() + bias
    q, k, v = x[:, :nq * d].view(N, nq, d), x[:, nq * d:(nq + nkv) * d].view(N, nkv, d), x[:, (nq + nkv) * d:].view(N, nkv, d)
    q, k = plain.rms_norm(q, qw, 1e-6), plain.rms_norm(k, kw, 1e-6)

    def rotate(t):
        c = torch.cat((cos, cos), -1)[:, None, :]
        s = torch.cat((sin, sin), -1)[:, None, :]
        head = t[..., :rot]
        return torch.cat((head * c + plain.rotate_half(head) * s, t[..., rot:]), dim=-1)

    q, k = rotate(q), rotate(k)
    t = tol(dtype, 1e-5, 5e-2)
    assert torch.allclose(work[:, :nq * d].float().view(N, nq, d), q, atol=t)
    for n in range(N):
        s = int(slots[n])
        if s < 0:
            continue
        assert torch.allclose(pages[s // page_size, 0, :, s % page_size].float(), k[n], atol=t)
        assert torch.allclose(pages[s // page_size, 1, :, s % page_size].float(), v[n], atol=t)
    untouched = torch.ones(pages_n * page_size, dtype=torch.bool)
    untouched[[int(s) for s in slots if s >= 0]] = False
    flat = pages.float().permute(0, 3, 1, 2, 4).reshape(pages_n * page_size, -1)
    assert float(flat[untouched].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [300, 296, 77])
def test_swiglu(dtype, width):
    gu = rnd(9, 2 * width, dtype=dtype, seed=9, scale=2.0)
    gu[0, :4] = torch.tensor([-30.0, 30.0, 0.0, -90.0], dtype=dtype, device=DEV)     # the ends of the sigmoid
    out = torch.empty(9, width, dtype=dtype, device=DEV)
    K().swiglu(gu, out)
    g, u = gu.float()[:, :width], gu.float()[:, width:]
    assert torch.isfinite(out).all()
    assert torch.allclose(out.float(), torch.nn.functional.silu(g) * u, atol=tol(dtype, 1e-6, 3e-2), rtol=tol(dtype, 1e-6, 1e-2))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,Kd", [(1, 130, 77), (70, 130, 77), (64, 64, 16), (3, 1000, 515)])
def test_gemm_simt(dtype, M, N, Kd):
    a, w = rnd(M, Kd, dtype=dtype, seed=10), rnd(N, Kd, dtype=dtype, seed=11)
    bias = rnd(N, seed=12)
    want = a.double() @ w.double().t() + bias.double()
    out = torch.empty(M, N, dtype=torch.float32, device=DEV) if dtype == torch.bfloat16 else torch.empty(M, N, device=DEV)
    K().gemm_simt(a, w, out, bias)
    assert torch.allclose(out.double(), want, atol=2e-4, rtol=1e-5)
    # a row's result does not depend on the other rows
    single = torch.empty(1, N, dtype=out.dtype, device=DEV)
    K().gemm_simt(a[M - 1:M], w, single, bias)
    assert torch.equal(single[0], out[M - 1])


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32], ids=["bf16", "f32out"])
@pytest.mark.parametrize("M,N,Kd", [(1, 130, 64), (8, 4096, 4096), (7, 100, 1048), (16, 6144, 520), (13, 331, 264),
                                     (9, 20000, 1032), (3, 17000, 256), (5, 20, 8)])
def test_gemm_skinny(out_dtype, M, N, Kd):
    x, w = rnd(M, Kd, dtype=torch.bfloat16, seed=13), rnd(N, Kd, dtype=torch.bfloat16, seed=14)
    want = x.double() @ w.double().t()
    out = torch.empty(M, N, dtype=out_dtype, device=DEV)
    K().gemm_skinny(x, w, out)
    scale = float(want.abs().max())
    assert float((out.double() - want).abs().max()) <= (2e-2 if out_dtype == torch.bfloat16 else 2e-4) * max(1.0, scale)
    # a row's result does not depend on the other rows, nor on their number
    for rows in (slice(M - 1, M), slice(0, 1)):
        single = torch.empty(1, N, dtype=out_dtype, device=DEV)
        K().gemm_skinny(x[rows], w, single)
        assert torch.equal(single[0], out[rows][0])
    with pytest.raises(K().KernelError, match="at most 16"):
        K().gemm_skinny(rnd(17, 16, dtype=torch.bfloat16), rnd(8, 16, dtype=torch.bfloat16),
                        torch.empty(17, 8, dtype=out_dtype, device=DEV))


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32], ids=["bf16", "f32out"])
@pytest.mark.parametrize("M,N,Kd", [(1, 130, 64), (8, 4096, 4096), (7, 100, 1048), (16, 6144, 520), (13, 331, 264),
                                     (33, 512, 128), (64, 3000, 1032), (128, 256, 64), (200, 331, 520),
                                     (2048, 1024, 4096), (300, 24, 72)])
def test_gemm_tcgen05(out_dtype, M, N, Kd):
    k_ = K()
    x, w = rnd(M, Kd, dtype=torch.bfloat16, seed=15), rnd(N, Kd, dtype=torch.bfloat16, seed=16)
    want = x.double() @ w.double().t()
    out = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
    k_.gemm_tc(x, w, out)
    torch.cuda.synchronize()
    k_.check_error_flag()
    scale = float(want.abs().max())
    assert float((out.double() - want).abs().max()) <= (2e-2 if out_dtype == torch.bfloat16 else 5e-4) * max(1.0, scale)
    # a row's result does not depend on the other rows of the call (same kernel variant)
    if M > 1 and M <= 16:
        single = torch.empty(1, N, dtype=out_dtype, device=DEV)
        k_.gemm_tc(x[M - 1:M], w, single)
        assert torch.equal(single[0], out[M - 1])


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M,N,Kd", [(1, 130, 64), (8, 4096, 4096), (5, 6144, 1024), (16, 1000, 192), (9, 331, 128),
                                    (3, 24576, 512), (8, 40000, 256), (2, 7, 64), (17, 4096, 256), (32, 5120, 512),
                                    (33, 1000, 192), (64, 4096, 128), (50, 4736, 128)])
def test_gemm_stream(M, N, Kd, out_dtype):
    """The weight-streaming kernel: row counts that give ragged shares per block, one and two 8-row tiles of
    x, several chunks of rows per block (N = 40000), fewer rows than blocks."""
    k_ = K()
    x, w = rnd(M, Kd, dtype=torch.bfloat16, seed=30), rnd(N, Kd, dtype=torch.bfloat16, seed=31)
    want = x.double() @ w.double().t()
    out = torch.empty(M, N, dtype=out_dtype, device=DEV)
    assert k_.gemm_stream_supports(M, N, Kd, Kd, Kd)
    k_.gemm_stream(x, w, out)
    k_.check_error_flag()
    scale = float(want.abs().max())
    assert torch.allclose(out.double(), want, atol=(2e-2 if out_dtype == torch.bfloat16 else 2e-4) * scale, rtol=0)
    # a row's result does not depend on the other rows
    single = torch.empty(1, N, dtype=out_dtype, device=DEV)
    k_.gemm_stream(x[M - 1:M], w, single)
    assert torch.equal(single[0], out[M - 1])


@pytest.mark.parametrize("M,I,Kd", [(1, 100, 64), (8, 12288, 4096), (5, 331, 128), (16, 3072, 1024), (3, 25600, 256)])
def test_gemm_stream_swiglu(M, I, Kd):
    """The fused gate/up product and activation: ragged shares per block, several chunks of rows per half."""
    k_ = K()
    x = rnd(M, Kd, dtype=torch.bfloat16, seed=40)
    w = rnd(2 * I, Kd, dtype=torch.bfloat16, seed=41, scale=0.5)
    assert k_.gemm_stream_swiglu_supports(M, I, Kd, Kd, Kd)
    out = torch.empty(M, I, dtype=torch.bfloat16, device=DEV)
    k_.gemm_stream_swiglu(x, w, out)
    k_.check_error_flag()
    y = x.double() @ w.double().t()
    want = torch.nn.functional.silu(y[:, :I]) * y[:, I:]
    assert torch.allclose(out.double(), want, atol=2e-2 * float(want.abs().max()), rtol=0)
    single = torch.empty(1, I, dtype=torch.bfloat16, device=DEV)
    k_.gemm_stream_swiglu(x[M - 1:M], w, single)
    assert torch.equal(single[0], out[M - 1])


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M,N,Kd", [(1, 130, 64), (8, 4096, 4096), (17, 6144, 1024), (16, 1000, 192), (33, 331, 128),
                                    (64, 24576, 512), (40, 40000, 256), (2, 7, 64), (64, 4096, 12288), (50, 5120, 256)])
def test_gemm_stream_tc(M, N, Kd, out_dtype):
    """The tcgen05 weight stream: row counts that leave a plane of W off the 1024-byte swizzle pattern (its
    descriptor carries the phase), 16, 32 and 64 rows of x, several chunks of rows per block."""
    k_ = K()
    x, w = rnd(M, Kd, dtype=torch.bfloat16, seed=50), rnd(N, Kd, dtype=torch.bfloat16, seed=51)
    want = x.double() @ w.double().t()
    out = torch.empty(M, N, dtype=out_dtype, device=DEV)
    assert k_.gemm_stream_tc_supports(M, N, Kd, Kd, Kd)
    k_.gemm_stream_tc(x, w, out)
    k_.check_error_flag()
    scale = float(want.abs().max())
    assert torch.allclose(out.double(), want, atol=(2e-2 if out_dtype == torch.bfloat16 else 2e-4) * scale, rtol=0)
    single = torch.empty(1, N, dtype=out_dtype, device=DEV)
    k_.gemm_stream_tc(x[M - 1:M], w, single)
    assert torch.equal(single[0], out[M - 1])


def test_gemm_stream_refuses_what_it_does_not_take():
    k_ = K()
    for M, N, Kd in [(64, 24576, 4096), (8, 100, 72), (65, 64, 64)]:      # too many accumulators, K no multiple of 64, rows
        assert not k_.gemm_stream_supports(M, N, Kd, Kd, Kd)
        x, w = rnd(M, Kd, dtype=torch.bfloat16, seed=1), rnd(N, Kd, dtype=torch.bfloat16, seed=2)
        with pytest.raises(k_.KernelError, match="gemm_stream"):
            k_.gemm_stream(x, w, torch.empty(M, N, dtype=torch.bfloat16, device=DEV))


def attention_reference(q, k, v, window, scale):
    """q [T, nq, d] at positions P..P+T-1 over keys k, v [S, nkv, d]; S = P + T."""
    T, nq, d = q.shape
    S, nkv, _ = k.shape
    G = nq // nkv
    kk, vv = k.repeat_interleave(G, dim=1), v.repeat_interleave(G, dim=1)
    scores = torch.einsum("tnd,snd->nts", q.double(), kk.double()) * scale
    qpos = torch.arange(S - T, S)[:, None]
    kpos = torch.arange(S)[None, :]
    mask = kpos > qpos
    if window:
        mask = mask | (kpos < qpos - window + 1)
    scores = scores.masked_fill(mask[None].to(scores.device), float("-inf"))
    return torch.einsum("nts,snd->tnd", torch.softmax(scores, dim=-1), vv.double()).float()


def run_paged(dtype, nq, nkv, d, page_size, requests, window=0, seed=0, boost=None, decode=False, uneven=False,
              segments=1):
    """requests: list of (context_before, new_tokens). Pages are handed out in a scrambled order."""
    k_ = K()
    gen = torch.Generator().manual_seed(seed)
    R = len(requests)
    total_pages = sum(-(-(p + t) // page_size) for p, t in requests) + 3
    order = torch.randperm(total_pages, generator=gen).tolist()
    pages = rnd(total_pages, 2, nkv, page_size, d, dtype=dtype, seed=seed + 1)      # stale data everywhere
    width = max(-(-(p + t) // page_size) for p, t in requests)
    tables = torch.full((R, width), -1, dtype=torch.int32)
    N = sum(t for _, t in requests)
    q = rnd(N, nq * d, dtype=dtype, seed=seed + 2)
    ks, vs, q_start, ctx = [], [], [0], []
    for r, (P, T) in enumerate(requests):
        S = P + T
        k, v = rnd(S, nkv, d, dtype=dtype, seed=seed + 10 + r), rnd(S, nkv, d, dtype=dtype, seed=seed + 50 + r)
        if boost is not None and r == boost[0]:
            # make one far key decisive for the last query of this request
            _, key_pos, head = boost
            kvh = head // (nq // nkv)
            qrow = q_start[-1] + T - 1
            direction = torch.nn.functional.normalize(rnd(d, seed=99), dim=0)
            q[qrow, head * d:(head + 1) * d] = (direction * 6 * math.sqrt(d) ** 0.5).to(dtype)
            k[key_pos, kvh] = (direction * 6 * math.sqrt(d) ** 0.5).to(dtype)
        for i in range(-(-S // page_size)):
            page = order.pop()
            tables[r, i] = page
            n = min(page_size, S - i * page_size)
            pages[page, 0, :, :n] = k[i * page_size:i * page_size + n].transpose(0, 1)
            pages[page, 1, :, :n] = v[i * page_size:i * page_size + n].transpose(0, 1)
        ks.append(k)
        vs.append(v)
        q_start.append(q_start[-1] + T)
        ctx.append(S)
    tpt = k_.tokens_per_attention_tile(nq, nkv, dtype, d, page_size)
    tile_req, tile_tok0, tile_seg, tile_slot = [], [], [], []
    for r, (_, T) in enumerate(requests):
        for t0 in range(0, T, tpt):
            # with segments: every tile as that many consecutive items that share its keys
            for k in range(segments):
                tile_req.append(r)
                tile_tok0.append(t0)
                tile_seg.append(k | segments << 8)
                tile_slot.append(len(tile_req) - 1 - k)
    dev = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)   # noqa: E731
    out = torch.zeros(N, nq * d, dtype=dtype, device=DEV)
    scale = d ** -0.5
    if decode:
        assert all(t == 1 for _, t in requests)
        k_.decode_attention(q, q.stride(0), out, pages, tables.to(DEV), dev(ctx), max(ctx), nq, nkv, d, page_size,
                            window, scale, uneven=uneven)
    else:
        shared = dict(tile_seg=dev(tile_seg), tile_slot=dev(tile_slot), places=len(tile_req)) if segments > 1 else {}
        k_.paged_attention(q, q.stride(0), out, pages, tables.to(DEV), dev(q_start), dev(ctx), dev(tile_req),
                           dev(tile_tok0), nq, nkv, d, page_size, window, scale, tpt, **shared)
    want = torch.cat([attention_reference(q[q_start[r]:q_start[r + 1]].float().view(-1, nq, d).cpu(), ks[r].float().cpu(),
                                          vs[r].float().cpu(), window, scale) for r in range(R)])
    return out.float().cpu().view(N, nq, d), want


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,page", [(4, 2, 16, 16), (6, 1, 32, 8), (9, 3, 48, 4), (32, 8, 128, 16), (5, 5, 80, 16),
                                           (40, 2, 64, 32)])
def test_paged_attention_mixed_batch(dtype, nq, nkv, d, page):
    got, want = run_paged(dtype, nq, nkv, d, page, [(0, 37), (130, 1), (63, 2), (64, 33), (5, 1), (0, 1)], seed=3)
    assert torch.allclose(got, want, atol=tol(dtype, 2e-5, 2e-2))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,page", [(4, 2, 16, 16), (6, 1, 32, 8), (9, 3, 48, 4), (32, 8, 128, 16), (5, 5, 80, 16),
                                           (40, 2, 64, 32), (16, 1, 256, 16), (16, 1, 128, 16), (8, 2, 128, 4)])
def test_decode_attention_split_keys(dtype, nq, nkv, d, page):
    # contexts on both sides of the 256-key ranges and of the 64-key tiles
    requests = [(0, 1), (255, 1), (256, 1), (700, 1), (63, 1), (64, 1), (1030, 1)]
    got, want = run_paged(dtype, nq, nkv, d, page, requests, seed=6, decode=True)
    assert torch.allclose(got, want, atol=tol(dtype, 2e-5, 2e-2))
    got_w, want_w = run_paged(dtype, nq, nkv, d, page, requests, window=300, seed=6, decode=True)
    assert torch.allclose(got_w, want_w, atol=tol(dtype, 2e-5, 2e-2))


@pytest.mark.parametrize("uneven", [False, True])
@pytest.mark.parametrize("nq,nkv,page", [(32, 8, 16), (8, 1, 8), (4, 4, 32), (6, 2, 64), (16, 2, 128)])
def test_decode_attention_head_size_128_streaming_kernel(nq, nkv, page, uneven):
    """Head size 128 in bfloat16 with up to 8 heads per group takes one of the two persistent TMA kernels (blocks of
    its own for every request, or all key ranges dealt out evenly): contexts on both sides of the 128-key ranges and
    of a warp's 32 keys, and enough requests that every block's ring of stages is filled several times over."""
    dtype = torch.bfloat16
    contexts = [0, 31, 32, 127, 128, 255, 256, 700, 63, 64, 1030, 5, 129, 511] * 3
    requests = [(c, 1) for c in contexts]
    got, want = run_paged(dtype, nq, nkv, 128, page, requests, seed=21, decode=True, uneven=uneven)
    assert torch.allclose(got, want, atol=2e-2)
    got_w, want_w = run_paged(dtype, nq, nkv, 128, page, requests, window=300, seed=22, decode=True, uneven=uneven)
    assert torch.allclose(got_w, want_w, atol=2e-2)
    K().check_error_flag()
    for key_pos in (3, 127, 128, 511, 698):
        got, want = run_paged(dtype, 8, 2, 128, 16, [(699, 1), (40, 1)], seed=4, boost=(0, key_pos, 5), decode=True,
                              uneven=uneven)
        assert torch.allclose(got, want, atol=3e-2), key_pos
        assert float(want[0, 5].abs().max()) > 0.5


@pytest.mark.parametrize("segments", [2, 3, 8])
def test_prefill_attention_head_size_128_items_share_a_tile(segments):
    """The tcgen05 kernel with every tile as several items that share its keys: each leaves its sums in global memory
    and the last to finish adds them up. Contexts with fewer key tiles than items (items without keys), a window
    that leaves some items nothing, one decisive key in an item in the middle; several launches in a row, since
    the counters must be zero again."""
    dtype = torch.bfloat16
    assert K().attention_max_segments(8, 2, dtype, 128, 16) >= 8
    requests = [(0, 37), (1130, 70), (63, 2), (300, 200), (5, 1), (700, 33)]
    for seed, window in ((41, 0), (42, 0), (43, 200)):
        boost = (1, 600, 5) if window == 0 else None
        got, want = run_paged(dtype, 8, 2, 128, 16, requests, window=window, seed=seed, boost=boost, segments=segments)
        assert torch.allclose(got, want, atol=3e-2), (seed, window, float((got - want).abs().max()))
    K().check_error_flag()
    with pytest.raises(Exception, match="whole tiles only"):
        run_paged(dtype, 4, 2, 64, 16, [(100, 40)], segments=2)


@pytest.mark.parametrize("contexts", [[40000, 10, 300, 129], [9000], [5], [3000, 2999, 3001, 1, 2, 3, 700, 700, 128],
                                      [20000] * 3 + [17] * 40, [511] * 150, [9000] + [40] * 530])
@pytest.mark.parametrize("uneven", [True, False])
def test_decode_attention_streaming_kernel_shares_long_requests(contexts, uneven):
    """The kernel for uneven batches deals the 128-key ranges of all requests out evenly: a request far longer than
    the others is shared by many blocks, whose sums the last of them to finish adds up. One decisive key in the long
    request, in a range of a block in the middle; several times in a row, since the blocks' counters must be zero
    again. The kernel for even batches takes the same batches, only slower, and those of more than 512 requests."""
    dtype = torch.bfloat16
    requests = [(c, 1) for c in contexts]
    key_pos = contexts[0] // 2
    for seed, window in ((31, 0), (32, 0), (33, 2500)):
        boost = (0, key_pos, 5) if window == 0 else None
        got, want = run_paged(dtype, 8, 2, 128, 32, requests, window=window, seed=seed, boost=boost, decode=True,
                              uneven=uneven)
        assert torch.allclose(got, want, atol=3e-2), (seed, window, float((got - want).abs().max()))
        if boost is not None:
            assert float(want[0, 5].abs().max()) > 0.5
    K().check_error_flag()


@pytest.mark.parametrize("dtype", DTYPES)
def test_decode_attention_finds_one_far_key(dtype):
    for key_pos in (3, 255, 256, 511, 698):
        got, want = run_paged(dtype, 8, 2, 64, 16, [(699, 1), (40, 1)], seed=4, boost=(0, key_pos, 5), decode=True)
        assert torch.allclose(got, want, atol=tol(dtype, 3e-5, 3e-2)), key_pos
        assert float(want[0, 5].abs().max()) > 0.5


@pytest.mark.parametrize("dtype", DTYPES)
def test_paged_attention_finds_one_far_key_among_hundreds(dtype):
    # decode over 700 keys: key 3 (first page) decides head 5; then key 511 (a page's last slot)
    for key_pos in (3, 511, 512, 699):
        got, want = run_paged(dtype, 8, 2, 64, 16, [(699, 1), (40, 8)], seed=4, boost=(0, key_pos, 5))
        assert torch.allclose(got, want, atol=tol(dtype, 3e-5, 3e-2)), key_pos
        assert float(want[0, 5].abs().max()) > 0.5      # the boosted key dominates: its value shows in the output


@pytest.mark.parametrize("nq,nkv,page", [(32, 8, 16), (4, 4, 8), (6, 2, 32), (7, 1, 64), (16, 1, 128), (12, 3, 16)])
def test_prefill_attention_head_size_128_tensor_memory_kernel(nq, nkv, page):
    """Head size 128 in bfloat16 takes the tcgen05 kernel: portions that cross several 128-key tiles, a
    portion that starts in the middle of a tile, single tokens, and a prompt shorter than one tile."""
    dtype = torch.bfloat16
    assert K().tokens_per_attention_tile(nq, nkv, dtype, 128, page) == 128 // (nq // nkv)
    requests = [(0, 300), (515, 130), (127, 2), (128, 1), (0, 1), (250, 7), (0, 129)]
    got, want = run_paged(dtype, nq, nkv, 128, page, requests, seed=11)
    assert torch.allclose(got, want, atol=2e-2)
    got_w, want_w = run_paged(dtype, nq, nkv, 128, page, requests, window=200, seed=12)
    assert torch.allclose(got_w, want_w, atol=2e-2)
    K().check_error_flag()


def test_prefill_attention_head_size_128_finds_one_far_key():
    for key_pos in (3, 127, 128, 511, 698):
        got, want = run_paged(torch.bfloat16, 8, 2, 128, 16, [(600, 100), (40, 8)], seed=4, boost=(0, key_pos, 5))
        assert torch.allclose(got, want, atol=3e-2), key_pos
        assert float(want[99, 5].abs().max()) > 0.5
    for window, offset in ((1, 0), (33, 0), (33, 1), (128, 0), (128, 1), (300, 1)):
        P, T = 450, 70
        key_pos = P + T - window - offset                   # offset 0: the oldest key inside; 1: the first outside
        got, want = run_paged(torch.bfloat16, 8, 2, 128, 16, [(P, T), (20, 5)], window=window, seed=5, boost=(0, key_pos, 1))
        assert torch.allclose(got, want, atol=3e-2), (window, offset)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [1, 7, 32, 33, 100])
def test_paged_attention_window_edge(dtype, window):
    # the key just inside and just outside the window of the last query are the decisive ones
    for offset in (0, 1):
        P, T = 150, 3
        key_pos = P + T - 1 - window + 1 - offset       # offset 0: the oldest key inside; 1: the first outside
        if key_pos < 0:
            continue
        got, want = run_paged(dtype, 4, 2, 32, 8, [(P, T), (20, 5)], window=window, seed=5, boost=(0, key_pos, 1))
        assert torch.allclose(got, want, atol=tol(dtype, 3e-5, 3e-2)), (window, offset)


def test_argmax_and_sampling_rows():
    k_ = K()
    from llm_pipeline_b200.sampling import Sampler, SamplingConfig, uniform_of
    V = 1531
    logits = rnd(6, V, seed=20, scale=3.0)
    logits[2, 77] = logits[2].max() + 1
    logits[2, 900] = logits[2, 77]                   # a tie: the lower index wins
    out = torch.empty(6, dtype=torch.int32, device=DEV)
    k_.argmax(logits, out)
    assert out.tolist() == logits.cpu().argmax(dim=-1).tolist() and out[2] == 77
    sampler = Sampler()
    configs = [SamplingConfig(temperature=0.0), SamplingConfig(temperature=0.7, top_k=0, top_p=1.0, seed=1),
               SamplingConfig(temperature=1.3, top_k=40, top_p=1.0, seed=2),
               SamplingConfig(temperature=0.9, top_k=50, top_p=0.9, seed=3),
               SamplingConfig(temperature=1.0, top_k=0, top_p=0.5, min_p=0.05, seed=4),
               SamplingConfig(temperature=0.8, top_k=200, top_p=0.95, typical_p=0.9, seed=5)]
    for step in range(12):
        got = sampler.sample_rows(logits, configs, [step] * 6).tolist()
        assert got[0] == int(logits[0].argmax())
        for r in range(1, 6):
            c = configs[r]
            probs = plain.filtered_probs(logits[r].cpu(), c.temperature, c.top_k, c.top_p, c.min_p, c.typical_p)
            u = uniform_of(c.seed, step)
            assert probs[got[r]] > 0, (r, step)
            cdf = torch.cumsum(probs.double(), 0)
            lo = float(cdf[got[r]] - probs[got[r]].double())
            assert lo - 1e-4 <= u <= float(cdf[got[r]]) + 1e-4, (r, step, u, lo, float(cdf[got[r]]))
    # a row's draw does not depend on the rows around it
    alone = sampler.sample_rows(logits[3:4], [configs[3]], [5]).tolist()[0]
    assert alone == sampler.sample_rows(logits, configs, [5] * 6).tolist()[3]
    # repetition penalty moves mass away from listed tokens
    cfg = SamplingConfig(temperature=0.0, repetition_penalty=50.0)
    top = int(logits[1].argmax())
    assert sampler.sample_rows(logits[1:2], [cfg], [0], [[top]]).tolist()[0] != top


def test_kernels_refuse_what_they_cannot_do():
    k_ = K()
    with pytest.raises(k_.KernelError, match="CUDA"):
        k_.embedding(torch.zeros(1, dtype=torch.int32), torch.zeros(2, 2), torch.zeros(1, 2))
    with pytest.raises(k_.KernelError, match="multiple of 16"):
        run_paged(torch.float32, 2, 1, 24, 8, [(0, 2)])
    with pytest.raises(k_.KernelError, match="float32 and bfloat16"):
        k_.swiglu(torch.zeros(2, 4, dtype=torch.float16, device=DEV), torch.zeros(2, 2, dtype=torch.float16, device=DEV))


@pytest.mark.parametrize("M,N,Kd,H", [(8, 4096, 4096, 4096), (1, 1024, 3072, 1024), (5, 5120, 256, 5120), (3, 192, 320, 192)])
def test_gemm_stream_between_norms(M, N, Kd, H):
    """The streaming product with the residual add and the RMSNorm around it folded in: as producer it adds into the
    float32 residual and leaves residual * norm weight and its blocks' sums of squares; as consumer it multiplies its
    result by the rows' factors. Together they give what the norm kernel between two plain products gives."""
    k_ = K()
    x, w = rnd(M, Kd, dtype=torch.bfloat16, seed=70), rnd(N, Kd, dtype=torch.bfloat16, seed=71, scale=0.05)
    residual = rnd(M, N, seed=72, scale=3.0)
    for norm_dtype in (torch.float32, torch.bfloat16):
        norm_w = (1 + 0.2 * rnd(N, seed=73)).to(norm_dtype)
        blocks = k_.gemm_stream_blocks(M, N, Kd, Kd, Kd)
        assert blocks > 0
        res = residual.clone()
        xw = torch.zeros(M, N, dtype=torch.bfloat16, device=DEV)
        sumsq = torch.full((blocks + 2, 8), 7.0, device=DEV)
        k_.gemm_stream_fused(x, w, None, residual=res, norm_weight=norm_w, xw=xw, out_sumsq=sumsq)
        want_res = residual.double() + x.double() @ w.double().t()
        assert torch.allclose(res.double(), want_res, atol=2e-3, rtol=1e-5)
        assert torch.equal(xw, (res * norm_w.float()).to(torch.bfloat16))
        assert torch.allclose(sumsq[:blocks, :M].sum(0).double(), (res.double() ** 2).sum(1), rtol=1e-5)
        assert float(sumsq[:blocks, M:].abs().max()) == 0.0 if M < 8 else True
        assert float(sumsq[blocks:].min()) == 7.0                    # rows beyond the blocks are not touched
        # the same launch again gives the same bits (sums in a fixed order)
        res2, xw2, sumsq2 = residual.clone(), torch.zeros_like(xw), torch.zeros_like(sumsq)
        k_.gemm_stream_fused(x, w, None, residual=res2, norm_weight=norm_w, xw=xw2, out_sumsq=sumsq2)
        assert torch.equal(res2, res) and torch.equal(sumsq2[:blocks], sumsq[:blocks])
    # consumer: a product of the rows that lack their factors, against the norm kernel and a plain product
    eps = 1e-6
    norm_w = (1 + 0.2 * rnd(N, seed=73))
    res = residual.clone()
    xw = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    blocks = k_.gemm_stream_blocks(M, N, Kd, Kd, Kd)
    sumsq = torch.empty(blocks, 8, device=DEV)
    k_.gemm_stream_fused(x, w, None, residual=res, norm_weight=norm_w, xw=xw, out_sumsq=sumsq)
    w2 = rnd(2 * 96, H, dtype=torch.bfloat16, seed=74, scale=0.05)
    assert N == H
    normed = plain.rms_norm(want_res.float(), norm_w, eps)
    want = normed.double() @ w2.double().t()
    out = torch.empty(M, w2.shape[0], dtype=torch.bfloat16, device=DEV)
    k_.gemm_stream_fused(xw, w2, out, in_sumsq=sumsq, in_parts=blocks, in_width=H, in_eps=eps)
    scale = float(want.abs().max())
    assert float((out.double() - want).abs().max()) <= 2e-2 * max(1.0, scale)
    # and with SwiGLU
    act = torch.empty(M, 96, dtype=torch.bfloat16, device=DEV)
    k_.gemm_stream_fused(xw, w2, act, glu=True, in_sumsq=sumsq, in_parts=blocks, in_width=H, in_eps=eps)
    want_act = torch.nn.functional.silu(want[:, :96]) * want[:, 96:]
    assert float((act.double() - want_act).abs().max()) <= 3e-2 * max(1.0, float(want_act.abs().max()))
    k_.check_error_flag()


def test_a_wait_that_runs_out_reaches_the_host_and_the_next_launch_works():
    """Every wait on a barrier in the TMA and tcgen05 kernels is bounded; a wait that runs out sets a word in mapped
    host memory and the kernel returns. Here the kernels' own wait gets a barrier that nothing completes and a small
    limit: it gives up, the host check raises, and the device goes on working (nothing faulted or hung)."""
    from llm_pipeline_b200.ops.kernels import KernelError
    k = K()
    torch.cuda.synchronize()
    k.check_error_flag()                                     # clean before
    assert k.bounded_wait_check(limit=1024)                  # the wait returned without completion
    torch.cuda.synchronize()
    with pytest.raises(KernelError, match="gave up waiting"):
        k.check_error_flag()
    k.check_error_flag()                                     # raising cleared the word
    x, w = rnd(8, 256, dtype=torch.bfloat16, seed=1), rnd(512, 256, dtype=torch.bfloat16, seed=2)
    out = torch.empty(8, 512, dtype=torch.float32, device=DEV)
    k.gemm_tc(x, w, out)                                     # a kernel with bounded waits of its own, right after
    torch.cuda.synchronize()
    k.check_error_flag()
    assert torch.allclose(out, x.float() @ w.float().t(), atol=1e-3, rtol=1e-3)
    with pytest.raises(KernelError):
        k.bounded_wait_check(limit=0)


@pytest.mark.parametrize("M,H,Q,I,QKV", [(8, 4096, 4096, 12288, 6144), (1, 1024, 2048, 3072, 4096), (5, 5120, 8192, 25600, 10240),
                                         (3, 192, 128, 320, 384), (8, 4096, 4096, 12288, 0)])
def test_gemm_stream_chain_gives_the_bits_of_its_products(M, H, Q, I, QKV):
    """Output projection (into the residual, next norm folded in) -> gate/up with SwiGLU -> down projection (into the
    residual) -> the next q/k/v projection as phases of one persistent launch, against the same four products launched
    one by one: the same bits everywhere, and the plain float32 reference within rounding. QKV = 0: three phases, the
    last one with plain rows."""
    k = K()
    attn = rnd(M, Q, dtype=torch.bfloat16, seed=1)
    w_o, w_gu = rnd(H, Q, dtype=torch.bfloat16, seed=2, scale=0.05), rnd(2 * I, H, dtype=torch.bfloat16, seed=3, scale=0.05)
    w_d = rnd(H, I, dtype=torch.bfloat16, seed=4, scale=0.05)
    w_qkv = rnd(QKV, H, dtype=torch.bfloat16, seed=5, scale=0.05) if QKV else None
    n1, n2 = (1 + 0.1 * rnd(H, seed=6)), (1 + 0.1 * rnd(H, seed=7))
    residual0 = rnd(M, H, seed=8)
    eps = 1e-6

    def run(chained):
        residual = residual0.clone()
        blocks = k.gemm_stream_blocks(M, H, Q, Q, Q)
        blocks_d = k.gemm_stream_blocks(M, H, I, I, I)
        xw1, ss1 = torch.empty(M, H, dtype=torch.bfloat16, device=DEV), torch.zeros(blocks, 8, device=DEV)
        act = torch.empty(M, I, dtype=torch.bfloat16, device=DEV)
        xw2, ss2 = torch.empty(M, H, dtype=torch.bfloat16, device=DEV), torch.zeros(blocks_d, 8, device=DEV)
        last = torch.empty(M, QKV, dtype=torch.bfloat16, device=DEV) if QKV else torch.empty(M, H, dtype=torch.bfloat16, device=DEV)
        calls = [(attn, w_o, None, dict(residual=residual, norm_weight=n1, xw=xw1, out_sumsq=ss1)),
                 (xw1, w_gu, act, dict(glu=True, in_sumsq=ss1, in_parts=blocks, in_width=H, in_eps=eps))]
        if QKV:
            calls += [(act, w_d, None, dict(residual=residual, norm_weight=n2, xw=xw2, out_sumsq=ss2)),
                      (xw2, w_qkv, last, dict(in_sumsq=ss2, in_parts=blocks_d, in_width=H, in_eps=eps))]
        else:
            calls += [(act, w_d, last, {})]
        if chained:
            phases = [k.chain_phase(x, w, out, **extras) for x, w, out, extras in calls]
            assert k.gemm_stream_chain_supports(phases, M)
            k.gemm_stream_chain(phases, M, torch.device(DEV))
        else:
            for x, w, out, extras in calls:
                k.gemm_stream_fused(x, w, out, **extras)
        torch.cuda.synchronize()
        k.check_error_flag()
        return residual, xw1, ss1, act, xw2, ss2, last

    one_by_one = run(False)
    for attempt in range(3):                                    # the counters of the chain are left zero: launch after launch
        chained = run(True)
        for name, a, b in zip(("residual", "xw1", "sumsq1", "act", "xw2", "sumsq2", "last"), one_by_one, chained):
            if QKV or name not in ("xw2", "sumsq2"):
                assert torch.equal(a, b), (name, attempt, float((a.float() - b.float()).abs().max()))
    # and the whole against plain float32 arithmetic on the same bfloat16 operands
    r1 = residual0 + attn.float() @ w_o.float().t()
    x1 = plain.rms_norm(r1, n1, eps)
    gu = x1 @ w_gu.float().t()
    a_ref = torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]
    d_ref = a_ref @ w_d.float().t()
    assert torch.allclose(chained[3].float(), a_ref, atol=3e-2 * float(a_ref.abs().max()), rtol=3e-2)
    if QKV:
        r2 = r1 + d_ref
        q_ref = plain.rms_norm(r2, n2, eps) @ w_qkv.float().t()
        assert torch.allclose(chained[0], r2, atol=3e-2 * float(r2.abs().max()))
        assert torch.allclose(chained[6].float(), q_ref, atol=4e-2 * float(q_ref.abs().max()))
    else:
        assert torch.allclose(chained[6].float(), d_ref, atol=3e-2 * float(d_ref.abs().max()))


@pytest.mark.parametrize("M,N,Kd", [(2048, 4096, 4096), (300, 1000, 520), (1, 64, 8), (77, 4104, 264)])
def test_library_product_adds_into_the_float32_residual(M, N, Kd):
    """The library's product with the float32 residual as its C operand: residual += x w^T with float32 sums, the
    product itself never rounded to bfloat16; refused (False, nothing touched) for other types or unaligned rows."""
    x = rnd(M, Kd, dtype=torch.bfloat16, seed=1, scale=0.5)
    w = rnd(N, Kd, dtype=torch.bfloat16, seed=2, scale=0.1)
    residual = rnd(M, N, seed=3)
    want = residual.double() + x.double() @ w.double().t()
    got = residual.clone()
    assert K().library_add_product(got, x, w)
    scale = float(want.abs().max())
    assert float((got.double() - want).abs().max()) <= 2e-6 * scale * max(1, Kd // 64)      # float32 sums over K
    # closer than adding the product rounded to bfloat16 would be
    rounded = residual.double() + (x.double() @ w.double().t()).to(torch.bfloat16).double()
    if Kd >= 264:
        assert float((got.double() - want).abs().max()) < float((rounded - want).abs().max())
    untouched = residual.clone()
    assert not K().library_add_product(untouched, x.float(), w)
    assert not K().library_add_product(untouched[:, 1:], x, w[1:])
    assert torch.equal(untouched, residual)


def test_mirostat_v2_follows_the_reference_arithmetic():
    """inference/sampling.py:240-279: the entropy of softmax(logits / T), the running value moved by -eta (H - tau), a
    draw among the int(exp(value)) most likely tokens while the value is positive. Entropy kernel against float64
    (also with removed tokens, at a vocabulary that is no power of two); five calls in a row against the same
    arithmetic done by hand, the draw being this library's seeded draw with that top-k."""
    import math
    from llm_pipeline_b200.sampling import Sampler, SamplingConfig
    V = 10007
    logits = rnd(3, V, seed=3, scale=2.0)
    logits[1, 17:4000] = float("-inf")
    for T in (1.0, 0.7, 0.0):
        z = logits.double() / (T if T > 0 else 1.0)
        p = torch.softmax(z, dim=-1)
        want = -(p * torch.where(p > 0, torch.log_softmax(z, dim=-1), torch.zeros_like(z))).sum(-1)
        got = K().entropy(logits, T)
        assert torch.allclose(got.double().cpu(), want.cpu(), atol=2e-5), (T, got, want)
    cfg = SamplingConfig(temperature=0.8, mirostat_tau=3.0, mirostat_eta=0.3, seed=11)
    sampler = Sampler(cfg)
    value, by_hand = None, None
    for step in range(5):
        row = rnd(1, V, seed=40 + step, scale=3.0)
        z = row.double() / 0.8
        p = torch.softmax(z, dim=-1)
        H = float(-(p * torch.log_softmax(z, dim=-1)).sum())
        by_hand = H if by_hand is None else by_hand
        by_hand -= 0.3 * (H - 3.0)
        k = max(1, int(math.exp(by_hand))) if by_hand > 0 else 0
        token, value = sampler.sample_mirostat_v2(row, previous_entropy=value, step=step)
        assert abs(value - by_hand) < 1e-4 and token.shape == (1,) and token.dtype == torch.int64
        assert int(token) in set(torch.topk(row[0], k).indices.tolist()) if k else True
        same = sampler.sample_rows(row, [SamplingConfig(temperature=0.8, top_k=k, top_p=1.0, seed=11)], [step])
        assert int(same[0]) == int(token)
    with pytest.raises(ValueError, match="one sequence"):
        sampler.sample_mirostat_v2(logits)
