"""Each kernel alone against a plain float32/float64 reference of the same operation,
at sizes other than the tiny models': real widths, sizes that are no power of two,
page edges, window edges, shuffled pages, and inputs made so that one far key decides
the result."""
import math

import pytest
import torch

import plain_qwen3 as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def F():
    from mini_llm_runtime_b200.ops import functions
    return functions


def status():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


def gen(seed):
    return torch.Generator().manual_seed(seed)


# ------------------------------------------------------------------ row-wise kernels
@pytest.mark.parametrize("rows,width,vocab", [(7, 100, 33), (64, 4096, 151936), (3, 5120 + 6, 1000)])
@pytest.mark.parametrize("wdtype", [torch.float32, torch.bfloat16])
def test_embed_gather(rows, width, vocab, wdtype):
    table = torch.randn(vocab, width, generator=gen(0)).to(wdtype).to(DEV)
    ids = torch.randint(0, vocab, (rows,), generator=gen(1), dtype=torch.int32).to(DEV)
    out, st = torch.full((rows, width), 7.0, device=DEV), status()
    F().embed_gather(table, ids, out, st)
    assert torch.equal(out, table[ids.long()].float()) and st.item() == 0
    ids[rows // 2] = vocab
    F().embed_gather(table, ids, out, st)
    assert st.item() == 1 and out[rows // 2].abs().sum() == 0


@pytest.mark.parametrize("rows,width", [(5, 64), (33, 4096), (4, 5120), (2, 1000), (3, 33)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("w_dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_with_residual_add(rows, width, out_dtype, w_dtype):
    h = torch.randn(rows, width, generator=gen(0)) * 3
    delta = torch.randn(rows, width, generator=gen(1))
    w = (1 + 0.1 * torch.randn(width, generator=gen(2))).to(w_dtype)
    eps = 1e-5
    want_h = h + delta
    want = P.rms_norm(want_h.double(), w.double(), eps)
    hd, out = h.clone().to(DEV), torch.empty(rows, width, dtype=out_dtype, device=DEV)
    F().rmsnorm(hd, w.to(DEV), eps, out, delta=delta.to(DEV))
    assert torch.equal(hd.cpu(), want_h)                       # the stream moved on
    tol = 1e-5 if out_dtype is torch.float32 else 1e-2
    assert torch.allclose(out.double().cpu(), want, rtol=tol, atol=tol)
    # Selected rows, stream untouched.
    idx = torch.tensor([rows - 1, 0], dtype=torch.int32, device=DEV)
    hd2, out2 = h.clone().to(DEV), torch.empty(2, width, dtype=out_dtype, device=DEV)
    F().rmsnorm(hd2, w.to(DEV), eps, out2, delta=delta.to(DEV), rows=idx, write_back=False)
    assert torch.equal(hd2.cpu(), h)
    assert torch.allclose(out2.double().cpu(), want[[rows - 1, 0]], rtol=tol, atol=tol)
    # Without a delta.
    F().rmsnorm(hd2, w.to(DEV), eps, out2[:1], rows=idx[:1])
    assert torch.allclose(out2[:1].double().cpu(), P.rms_norm(h[rows - 1:].double(), w.double(), eps), rtol=tol, atol=tol)


@pytest.mark.parametrize("width", [4096, 2048, 1000, 8192])
def test_rmsnorm_does_not_depend_on_how_many_rows_a_launch_has(width):
    """A row's result is the same bits whether it is normed alone or among hundreds."""
    h = torch.randn(200, width, generator=gen(3)) * 2
    delta = torch.randn(200, width, generator=gen(4))
    w = (1 + 0.1 * torch.randn(width, generator=gen(5)))
    for out_dtype in (torch.float32, torch.bfloat16):
        many, few = torch.empty(200, width, dtype=out_dtype, device=DEV), torch.empty(3, width, dtype=out_dtype, device=DEV)
        hd = h.clone().to(DEV)
        F().rmsnorm(hd, w.to(DEV), 1e-6, many, delta=delta.to(DEV))
        hd2 = h[:3].clone().to(DEV)
        F().rmsnorm(hd2, w.to(DEV), 1e-6, few, delta=delta[:3].contiguous().to(DEV))
        assert torch.equal(many[:3], few) and torch.equal(hd[:3], hd2)
        want = P.rms_norm((h + delta).double(), w.double(), 1e-6)
        tol = 1e-5 if out_dtype is torch.float32 else 1e-2
        assert torch.allclose(many.double().cpu(), want, rtol=tol, atol=tol)


def test_consumers_add_up_partial_sums():
    """A product whose K was cut into ranges leaves float32 partial sums; the norm, the
    gate and the q/k kernel add them up (in order) as they read them."""
    from mini_llm_runtime_b200.parts.rotary import rotation_table
    S, M, H = 3, 5, 96
    parts = torch.randn(S, M, H, generator=gen(0))
    h = torch.randn(M, H, generator=gen(1))
    w = (1 + 0.1 * torch.randn(H, generator=gen(2)))
    total = (parts[0] + parts[1]) + parts[2]
    for width in (96, 70):                           # the register-cached kernel and the plain one
        hd, out = h[:, :width].contiguous().to(DEV), torch.empty(M, width, device=DEV)
        F().rmsnorm(hd, w[:width].contiguous().to(DEV), 1e-5, out, delta=parts[:, :, :width].contiguous().to(DEV))
        want_h = h[:, :width] + total[:, :width]
        assert torch.equal(hd.cpu(), want_h)
        assert torch.allclose(out.cpu(), P.rms_norm(want_h, w[:width], 1e-5), atol=1e-5, rtol=1e-5)
    # The gate.
    I = 40
    gu = torch.randn(S, M, 2 * I, generator=gen(3))
    act = torch.empty(M, I, dtype=torch.bfloat16, device=DEV)
    F().swiglu(gu.to(DEV), act)
    t = (gu[0] + gu[1]) + gu[2]
    want = t[:, :I] / (1 + torch.exp(-t[:, :I])) * t[:, I:]
    assert torch.allclose(act.float().cpu(), want, atol=2e-2, rtol=2e-2)
    # q/k norm, rotation and cache write from partial sums equal the same from their sum.
    Hq, Hkv, D, page = 4, 2, 64, 8
    segs = [(3, 4), (0, 2)]
    rows = 6
    qkv_parts = torch.randn(S, rows, (Hq + 2 * Hkv) * D, generator=gen(4))
    summed = ((qkv_parts[0] + qkv_parts[1]) + qkv_parts[2])
    positions, seg_of_row, info = segments_meta(segs)
    table_cs = rotation_table(1e4, D, 32).to(DEV)
    wq, wk = torch.ones(D, device=DEV), torch.ones(D, device=DEV)
    results = []
    for use_parts in (True, False):
        cache, table = make_cache([(torch.zeros(s + c, Hkv, D), torch.zeros(s + c, Hkv, D)) for s, c in segs], page,
                                  torch.float32, seed=1)
        qkv = torch.zeros(rows, (Hq + 2 * Hkv) * D, device=DEV) if use_parts else summed.to(DEV)
        F().qk_norm_rope_cache(qkv, Hq, Hkv, D, wq, wk, 1e-5, table_cs, positions, seg_of_row, table, page, cache, True,
                               status(), partials=qkv_parts.to(DEV) if use_parts else None)
        results.append((qkv[:, :(Hq + Hkv) * D].cpu(), torch.nan_to_num(cache).cpu()))
    assert torch.equal(results[0][0], results[1][0]) and torch.equal(results[0][1], results[1][1])


@pytest.mark.parametrize("rows,inter", [(3, 176), (17, 12288), (1, 7)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu(rows, inter, dtype):
    gu = (torch.randn(rows, 2 * inter, generator=gen(0)) * 3).to(dtype)
    out = torch.empty(rows, inter, dtype=dtype, device=DEV)
    F().swiglu(gu.to(DEV), out)
    g, u = gu[:, :inter].double(), gu[:, inter:].double()
    want = g / (1 + torch.exp(-g)) * u
    tol = 1e-6 if dtype is torch.float32 else 1e-2
    assert torch.allclose(out.double().cpu(), want, rtol=tol, atol=tol)


@pytest.mark.parametrize("M,N,K", [(1, 64, 64), (5, 100, 37), (64, 64, 16), (65, 130, 129), (3, 515, 80), (130, 300, 4096)])
def test_gemm_f32_is_true_float32_and_independent_of_batching(M, N, K):
    a = torch.randn(M, K, generator=gen(0))
    w = torch.randn(N, K, generator=gen(1))
    out = torch.empty(M, N, device=DEV)
    F().gemm_f32(a.to(DEV), w.to(DEV), out)
    want = a.double() @ w.double().T
    # float32 products and sums: error ~ sqrt(K) * 2^-24 relative to the magnitudes summed.
    bound = 2e-7 * math.sqrt(K) * (a.abs().double() @ w.abs().double().T) + 1e-6
    assert ((out.double().cpu() - want).abs() <= bound).all()
    # The same row alone gives the same bits.
    alone = torch.empty(1, N, device=DEV)
    F().gemm_f32(a[M - 1:].to(DEV), w.to(DEV), alone)
    assert torch.equal(alone[0], out[M - 1])
    # A strided view of a wider buffer works.
    wide = torch.zeros(M, K + 8, device=DEV)
    wide[:, :K] = a.to(DEV)
    out2 = torch.empty(M, N, device=DEV)
    F().gemm_f32(wide[:, :K], w.to(DEV), out2)
    assert torch.equal(out2, out)


@pytest.mark.parametrize("M,N,K", [(1, 64, 64), (8, 4096, 4096), (3, 100, 96), (16, 515, 1056), (64, 300, 200), (65, 256, 64),
                                   (128, 256, 4096), (200, 515, 136), (2048, 6144, 4096), (300, 48, 12288), (129, 24, 72)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_bf16_tcgen05(M, N, K, out_dtype):
    x = (torch.randn(M, K, generator=gen(0)) * 0.5).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=gen(1)) * 0.1).to(torch.bfloat16).to(DEV)
    want = (x.float() @ w.float().T).double()         # exact products of bf16 values, float32 sums
    out = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
    st = status()
    F().gemm_bf16_tcgen05(x, w, out, st)
    assert st.item() == 0
    tol = 2e-2 if out_dtype is torch.bfloat16 else 1e-3
    assert torch.isfinite(out.float()).all()
    assert torch.allclose(out.double(), want, atol=tol * (1 + want.abs().max().item()), rtol=tol), \
        f"max diff {(out.double() - want).abs().max():.3e}"
    # Operands that are views with wider row strides.
    wide = torch.zeros(M, K + 64, dtype=torch.bfloat16, device=DEV)
    wide[:, :K] = x
    out2 = torch.empty_like(out)
    F().gemm_bf16_tcgen05(wide[:, :K], w, out2, st)
    assert torch.equal(out2, out)
    # K cut into ranges: the slices add up to the product.
    if K >= 256 and out_dtype is torch.float32:
        for splits in (2, 3):
            parts = torch.full((splits, M, N), float("nan"), device=DEV)
            F().gemm_bf16_tcgen05(x, w, parts, st)
            assert st.item() == 0
            assert torch.allclose(parts.double().sum(0), want, atol=tol * (1 + want.abs().max().item()), rtol=tol)


@pytest.mark.parametrize("M", [1, 2, 3, 5, 8])
@pytest.mark.parametrize("N,K", [(512, 264), (4096, 4096), (6144, 1024), (301, 96), (2, 8), (100, 12288), (300, 5120)])
def test_gemv_bf16_and_what_it_folds_in(M, N, K):
    """The few-row product on the CUDA cores: plain, added into the float32 stream, with the RMS norm of
    the stream (all rows, or indexed rows) as its prologue; odd row counts and widths that are no power of two."""
    x = (torch.randn(M, K, generator=gen(1)) * 0.7).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=gen(2)) * 0.05).to(torch.bfloat16)
    want = x.double() @ w.double().T
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    out32 = torch.full((M, N), float("nan"), device=DEV)
    native = __import__("mini_llm_runtime_b200.ops.native", fromlist=["x"])
    if native.module("gemv_bf16").mlr_gemv_bf16_fits(M, K):
        F().gemv_bf16(w.to(DEV), x.to(DEV), out, "bf16")
        assert torch.allclose(out.cpu().double(), want, atol=2e-2, rtol=2e-2)
        F().gemv_bf16(w.to(DEV), x.to(DEV), out32, "f32")
        assert torch.allclose(out32.cpu().double(), want, atol=1e-4, rtol=1e-4)
    else:
        # Eight rows of 12288 values leave no room for the ring of weights: refused, not wrong (a product that
        # adds into the stream, below, is cut along K instead).
        assert M * K * 2 > 150 * 1024
        with pytest.raises(Exception, match="do not fit shared memory"):
            F().gemv_bf16(w.to(DEV), x.to(DEV), out, "bf16")
    h = torch.randn(M, N, generator=gen(3))
    stream = h.clone().to(DEV)
    F().gemv_bf16(w.to(DEV), x.to(DEV), stream, "add_f32")
    assert torch.allclose(stream.cpu().double(), h.double() + want, atol=1e-4, rtol=1e-4)
    if K % 4 == 0 and M * K <= 8 * 4096:
        # The norm of the stream as the prologue, against the norm kernel followed by the plain product.
        rows_of_stream = 9
        hs = torch.randn(rows_of_stream, K, generator=gen(4)) * 3
        nw = (1 + 0.1 * torch.randn(K, generator=gen(5))).to(torch.bfloat16)
        index = torch.tensor([5, 0, 6, 2, 2, 1, 3, 4][:M], dtype=torch.int32)
        for rows in (None, index):
            source = hs[:M] if rows is None else hs[rows.long()]
            normed = P.rms_norm(source, nw.float(), 1e-5).to(torch.bfloat16)
            want_n = normed.double() @ w.double().T
            got = torch.full((M, N), float("nan"), device=DEV)
            F().gemv_bf16(w.to(DEV), hs.to(DEV), got, "f32", norm_weight=nw.to(DEV), eps=1e-5,
                          rows=rows.to(DEV) if rows is not None else None)
            assert torch.allclose(got.cpu().double(), want_n, atol=3e-2, rtol=3e-2), (got.cpu().double() - want_n).abs().max()


@pytest.mark.parametrize("M,inter,K", [(1, 256, 128), (4, 12288, 4096), (3, 300, 104), (8, 1000, 512), (8, 640, 5120)])
def test_gemv_bf16_gate(M, inter, K):
    """silu(gate) * up in the epilogue, over the stacked operand the feed-forward keeps (blocks of 128 gate
    rows and their up rows, padded with zero rows)."""
    x = torch.randn(M, K, generator=gen(1)).to(torch.bfloat16)
    wg = (torch.randn(inter, K, generator=gen(2)) * 0.08).to(torch.bfloat16)
    wu = (torch.randn(inter, K, generator=gen(3)) * 0.08).to(torch.bfloat16)
    stacked = F().interleave_gate_up(wg.to(DEV), wu.to(DEV))
    g, u = x.double() @ wg.double().T, x.double() @ wu.double().T
    want = (g / (1 + torch.exp(-g))) * u
    out = torch.full((M, stacked.shape[0] // 2), float("nan"), dtype=torch.bfloat16, device=DEV)
    F().gemv_bf16(stacked, x.to(DEV), out, "silu_gate")
    got = out.cpu().double()
    assert torch.allclose(got[:, :inter], want, atol=2e-2, rtol=2e-2) and (got[:, inter:] == 0).all()


def test_gemv_bf16_refuses_what_it_cannot_do():
    x = torch.zeros(9, 64, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(128, 64, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(Exception, match="1 to 8 rows"):
        F().gemv_bf16(w, x, torch.empty(9, 128, dtype=torch.bfloat16, device=DEV))
    with pytest.raises(Exception, match="multiple of 8"):
        F().gemv_bf16(w[:, :60].contiguous(), x[:1, :60].contiguous(), torch.empty(1, 128, dtype=torch.bfloat16, device=DEV))
    with pytest.raises(Exception, match="multiple of 256"):
        F().gemv_bf16(w, x[:1], torch.empty(1, 64, dtype=torch.bfloat16, device=DEV), "silu_gate")
    big = torch.zeros(8, 65536, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(Exception, match="do not fit shared memory"):
        F().gemv_bf16(torch.zeros(8, 65536, dtype=torch.bfloat16, device=DEV), big, torch.empty(8, 8, dtype=torch.bfloat16, device=DEV))
    # ... but a product that adds into the stream is cut along K until its activations fit
    stream = torch.zeros(8, 8, device=DEV)
    F().gemv_bf16(torch.ones(8, 65536, dtype=torch.bfloat16, device=DEV), torch.ones(8, 65536, dtype=torch.bfloat16, device=DEV), stream, "add_f32")
    assert (stream == 65536).all()


@pytest.mark.parametrize("M,H,I,QKV", [(8, 512, 6400, 640), (4, 264, 10240, 300), (1, 4096, 12288, 6144), (8, 384, 768, 128), (3, 256, 768, 384)])
def test_gemv_bf16_layer_with_parts_and_prepared_norms(M, H, I, QKV):
    """The four products of a layer as a decode step launches them: o_proj adds into the stream and leaves the next
    norm half done (the stream times the norm's weight as bfloat16, sums of squares per 16 rows), gate/up takes that,
    down adds (cut along K into parts of at most 4096 values) and
    prepares the q/k/v product's norm.  Against float64 and against the same products with the norm as a prologue;
    the same bits on every run."""
    g = lambda seed, *shape: (torch.randn(*shape, generator=gen(seed)) * 0.04).to(torch.bfloat16).to(DEV)
    w_o, w_down, w_qkv = g(1, H, H), g(2, H, I), g(3, QKV, H)
    w_gate_up = F().interleave_gate_up(g(4, I, H), g(5, I, H))
    attn = g(6, M, H)
    norm1 = (1 + 0.1 * torch.randn(H, generator=gen(7))).to(torch.bfloat16).to(DEV)
    norm2 = (1 + 0.1 * torch.randn(H, generator=gen(8))).to(torch.float32).to(DEV)
    stream0 = torch.randn(M, H, generator=gen(9)).to(DEV)
    native = __import__("mini_llm_runtime_b200.ops.native", fromlist=["x"])
    parts = native.module("gemv_bf16").mlr_gemv_bf16_parts
    assert parts(M, I) == -(-I // 4096) and parts(M, H) == 1          # parts of at most 4096 values: a lane keeps their activations in registers
    st = status()

    def layer(prepare):
        h = stream0.clone()
        act = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=DEV)
        qkv = torch.full((M, QKV), float("nan"), dtype=torch.bfloat16, device=DEV)
        if prepare:
            side = torch.full((M, H), float("nan"), dtype=torch.bfloat16, device=DEV)
            squares = torch.full(((H + 15) // 16, 8), float("nan"), device=DEV)
            F().gemv_bf16_add_prepare(w_o, attn, h, norm1, side, squares, st)
            F().gemv_bf16_prepared(w_gate_up, side, squares, 1e-6, act, "silu_gate", st)
            F().gemv_bf16_add_prepare(w_down, act, h, norm2, side, squares, st)
            F().gemv_bf16_prepared(w_qkv, side, squares, 1e-6, qkv, "bf16", st)
        else:
            F().gemv_bf16(w_o, attn, h, "add_f32", status=st)
            F().gemv_bf16(w_gate_up, h, act, "silu_gate", norm_weight=norm1, eps=1e-6, status=st)
            F().gemv_bf16(w_down, act, h, "add_f32", status=st)
            F().gemv_bf16(w_qkv, h, qkv, "bf16", norm_weight=norm2, eps=1e-6, status=st)
        assert st.item() == 0
        return h, act, qkv

    first, again, plain = layer(True), layer(True), layer(False)
    for a, b in zip(first, again):
        assert torch.equal(a, b)
    # float64 from the same bfloat16 roundings of the activations that the kernel makes: it rounds the stream
    # times the norm's weight and multiplies the finished sums by 1/rms.
    wd = lambda t: t.cpu().double()

    def normed(h, weight):
        rounded = (h.float() * weight.cpu().float()).to(torch.bfloat16).double()
        return rounded / torch.sqrt((h.double() ** 2).mean(-1, keepdim=True) + 1e-6)

    h1 = wd(stream0) + wd(attn) @ wd(w_o).T
    both = (normed(h1, norm1) @ wd(w_gate_up).T).view(M, -1, 2, 128)
    gate, up = both[:, :, 0].reshape(M, -1), both[:, :, 1].reshape(M, -1)
    act = ((gate / (1 + torch.exp(-gate))) * up)
    for got in (first, plain):
        assert torch.allclose(wd(got[1]), act, atol=2e-2, rtol=2e-2), (wd(got[1]) - act).abs().max()
        h2 = h1 + wd(got[1]) @ wd(w_down).T                       # from the activations the kernel rounded
        assert torch.allclose(wd(got[0]), h2, atol=1e-3, rtol=1e-3), (wd(got[0]) - h2).abs().max()
        want_qkv = normed(got[0].cpu(), norm2) @ wd(w_qkv).T
        assert torch.allclose(wd(got[2]), want_qkv, atol=3e-2, rtol=3e-2), (wd(got[2]) - want_qkv).abs().max()



def test_gemm_bf16_tcgen05_every_tile_width():
    x = (torch.randn(400, 512, generator=gen(0)) * 0.5).to(torch.bfloat16).to(DEV)
    w = (torch.randn(700, 512, generator=gen(1)) * 0.1).to(torch.bfloat16).to(DEV)
    want = x.float() @ w.float().T
    for tile in (16, 32, 64, 128, 256):
        out = torch.full((400, 700), float("nan"), dtype=torch.float32, device=DEV)
        st = status()
        F().gemm_bf16_tcgen05(x, w, out, st, tile_q=tile)
        assert st.item() == 0 and torch.allclose(out, want, atol=1e-2, rtol=1e-3), tile
    from mini_llm_runtime_b200.ops.native import KernelError
    with pytest.raises(KernelError, match="K % 8"):
        F().gemm_bf16_tcgen05(x[:, :100].contiguous(), w[:, :100].contiguous(), torch.empty(400, 700, device=DEV), status())


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (257, 512, 4096), (300, 700, 136), (1000, 1032, 520), (2048, 6144, 4096),
                                   (130, 24, 72), (600, 256, 12288)])
def test_gemm_bf16_tcgen05_pair_and_its_epilogues(M, N, K):
    """The two-SM product: plain stores, the add into a float32 matrix, and the SiLU gate over
    interleaved gate/up rows, beside float32 products of the same bfloat16 values."""
    x = (torch.randn(M, K, generator=gen(0)) * 0.5).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=gen(1)) * 0.1).to(torch.bfloat16).to(DEV)
    want = x.float() @ w.float().T
    scale = 1 + want.abs().max().item()
    st = status()
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    F().gemm_bf16_tcgen05_pair(x, w, out, st, "bf16")
    assert st.item() == 0 and torch.allclose(out.float(), want, atol=2e-2 * scale, rtol=2e-2)
    out32 = torch.full((M, N), float("nan"), device=DEV)
    F().gemm_bf16_tcgen05_pair(x, w, out32, st, "f32")
    assert st.item() == 0 and torch.allclose(out32, want, atol=1e-3 * scale, rtol=1e-3)
    # Adding into a matrix: one float32 rounding on top of the plain result, and nothing outside.
    wide = torch.randn(M + 1, N + 8, generator=gen(2)).to(DEV)
    before = wide.clone()
    F().gemm_bf16_tcgen05_pair(x, w, wide[:M, :N], st, "add_f32")
    assert st.item() == 0 and torch.equal(wide[:M, :N], before[:M, :N] + out32)
    assert torch.equal(wide[M:], before[M:]) and torch.equal(wide[:, N:], before[:, N:])
    # Operands that are views with wider row strides.
    padded = torch.zeros(M, K + 64, dtype=torch.bfloat16, device=DEV)
    padded[:, :K] = x
    again = torch.empty_like(out32)
    F().gemm_bf16_tcgen05_pair(padded[:, :K], w, again, st, "f32")
    assert torch.equal(again, out32)
    # The gate: w as gate rows then up rows, interleaved in blocks of 128.
    if N % 2 == 0:
        inter = N // 2
        stacked = F().interleave_gate_up(w[:inter], w[inter:])
        inner = stacked.shape[0] // 2
        assert inner % 128 == 0 and inner - inter < 128
        act = torch.full((M, inner), float("nan"), dtype=torch.bfloat16, device=DEV)
        F().gemm_bf16_tcgen05_pair(x, stacked, act, st, "silu_gate")
        g, u = out[:, :inter].float(), out[:, inter:].float()        # the bfloat16 gate and up, as the unfused path has them
        gated = g / (1 + torch.exp(-g)) * u
        assert st.item() == 0 and torch.allclose(act[:, :inter].float(), gated, atol=1e-2 * (1 + gated.abs().max().item()), rtol=2e-2)
        assert (act[:, inter:] == 0).all()
        # The kernel that applies the gate to a stored product reads the same interleaving.
        product = torch.empty(M, 2 * inner, dtype=torch.bfloat16, device=DEV)
        F().gemm_bf16_tcgen05_pair(x, stacked, product, st, "bf16")
        unfused = torch.empty(M, inner, dtype=torch.bfloat16, device=DEV)
        F().swiglu(product, unfused, 128)
        assert torch.allclose(unfused.float(), act.float(), atol=1e-2 * (1 + gated.abs().max().item()), rtol=2e-2)


def test_gemm_bf16_tcgen05_pair_refuses_what_it_cannot_do():
    from mini_llm_runtime_b200.ops.native import KernelError
    x = torch.zeros(300, 100, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(512, 100, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(KernelError, match="K % 8"):
        F().gemm_bf16_tcgen05_pair(x, w, torch.empty(300, 512, dtype=torch.bfloat16, device=DEV), status(), "bf16")
    x, w = x[:, :96].contiguous(), w[:, :96].contiguous()
    with pytest.raises(KernelError, match="does not fit"):
        F().gemm_bf16_tcgen05_pair(x, w, torch.empty(300, 512, device=DEV), status(), "bf16")
    with pytest.raises(KernelError, match="256"):
        F().gemm_bf16_tcgen05_pair(x, w[:300], torch.empty(300, 150, dtype=torch.bfloat16, device=DEV), status(), "silu_gate")


@pytest.mark.parametrize("rows,inter,block", [(3, 256, 128), (5, 384, 128), (2, 48, 16), (4, 21, 7)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu_over_interleaved_blocks(rows, inter, block, dtype):
    gu = (torch.randn(rows, 2 * inter, generator=gen(0)) * 3).to(dtype)
    blocks = gu.view(rows, inter // block, 2, block).double()
    g, u = blocks[:, :, 0].reshape(rows, inter), blocks[:, :, 1].reshape(rows, inter)
    want = g / (1 + torch.exp(-g)) * u
    tol = 1e-6 if dtype is torch.float32 else 1e-2
    out = torch.empty(rows, inter, dtype=dtype, device=DEV)
    F().swiglu(gu.to(DEV), out, block)
    assert torch.allclose(out.double().cpu(), want, rtol=tol, atol=tol)
    # From partial sums.
    parts = torch.stack([gu.float() * 0.25, gu.float() * 0.75]).to(DEV)
    F().swiglu(parts, out, block)
    assert torch.allclose(out.double().cpu(), want, rtol=tol, atol=tol)


# ------------------------------------------------------------------ paged cache helpers
def stored_row(x, dtype):
    """Rows [T, Hkv, D] as the cache stores them: bfloat16 caches with a head size of 64,
    128 or 256 keep the 16-byte chunk c of the token at position p at chunk c ^ (p & 7);
    every other cache keeps rows as they are.  (The permutation is its own inverse.)"""
    T, _, D = x.shape
    if dtype is not torch.bfloat16 or D not in (64, 128, 256):
        return x
    col = torch.arange(D)[None, None, :] ^ ((torch.arange(T) & 7) << 3)[:, None, None]
    return torch.gather(x, 2, col.expand_as(x))


def make_cache(kvs, page_size, dtype, seed=0, extra_pages=3):
    """kvs: list of (k, v) [T, Hkv, D] per request.  Returns cache [pages, 2, Hkv, ps, D]
    filled with NaN except the given tokens, on shuffled pages, and the block table."""
    Hkv, D = kvs[0][0].shape[1:]
    kvs = [(stored_row(k, dtype), stored_row(v, dtype)) for k, v in kvs]
    blocks = [-(-k.shape[0] // page_size) for k, _ in kvs]
    num_pages = sum(blocks) + extra_pages
    order = torch.randperm(num_pages, generator=gen(seed)).tolist()
    cache = torch.full((num_pages, 2, Hkv, page_size, D), float("nan"), dtype=dtype)
    table = torch.full((len(kvs), max(blocks)), -1, dtype=torch.int32)
    for i, (k, v) in enumerate(kvs):
        for b in range(blocks[i]):
            page = order.pop()
            n = min(page_size, k.shape[0] - b * page_size)
            cache[page, 0, :, :n] = k[b * page_size:b * page_size + n].transpose(0, 1).to(dtype)
            cache[page, 1, :, :n] = v[b * page_size:b * page_size + n].transpose(0, 1).to(dtype)
            table[i, b] = page
    return cache.to(DEV), table.to(DEV)


def segments_meta(segments):
    """segments: list of (start, count).  Returns positions, segment_of_row, segment_info."""
    pos, seg, info, row = [], [], [], 0
    for i, (start, count) in enumerate(segments):
        pos += list(range(start, start + count))
        seg += [i] * count
        info.append([row, count, start, i])
        row += count
    t = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    return t(pos), t(seg), t(info)


def fast_plain_attention(q, k, v, start, window, scale):
    """Dense float64 version of the same definition (the loop version is slow for
    thousands of keys): q [count, Hq, D], k, v [T, Hkv, D]."""
    count, Hq, D = q.shape
    T, Hkv = k.shape[0], k.shape[1]
    g = Hq // Hkv
    qd, kd, vd = q.double(), k.double().repeat_interleave(g, 1), v.double().repeat_interleave(g, 1)
    s = torch.einsum("qhd,thd->hqt", qd, kd) * scale
    pos = torch.arange(start, start + count)[:, None]
    t = torch.arange(T)[None, :]
    mask = (t > pos) | ((t < pos - window + 1) if window else torch.zeros_like(t, dtype=torch.bool))
    s = s.masked_fill(mask[None], float("-inf"))
    return torch.einsum("hqt,thd->qhd", torch.softmax(s, -1), vd)


def test_dense_reference_equals_the_plain_loop():
    q, k, v = (torch.randn(40, h, 16, generator=gen(i)) for i, h in ((0, 6), (1, 2), (2, 2)))
    for window in (None, 7):
        a = P.causal_attention(q, k, v, window)
        b = fast_plain_attention(q, k, v, 0, window or 0, 1 / 4.0)
        assert torch.allclose(a.double(), b, atol=1e-5)


ATTENTION_CASES = [
    # Hq, Hkv, D, page, [(context before, new tokens)], window
    (4, 2, 16, 4, [(0, 33)], 0),
    (6, 3, 32, 8, [(0, 1), (16, 1), (17, 2), (40, 77)], 0),
    (5, 1, 48, 16, [(100, 3), (0, 70), (39, 1), (40, 1), (41, 1)], 40),
    (32, 8, 128, 16, [(127, 1), (128, 1), (129, 1), (15, 1), (16, 1), (2047, 1)], 0),
    (32, 8, 128, 16, [(0, 129), (1536, 64), (63, 2)], 0),
    (16, 8, 128, 64, [(300, 200), (5, 1)], 128),
    (8, 8, 64, 1, [(10, 20), (70, 1)], 0),
    (16, 1, 256, 32, [(90, 40), (200, 1)], 100),
    (14, 2, 80, 16, [(64, 64), (500, 2), (1000, 1)], 0),
]


def run_attention_case(dtype, kernel, case, seed):
    Hq, Hkv, D, page, segs, window = case
    scale = 1 / math.sqrt(D)
    kvs, qs, wants = [], [], []
    for i, (before, count) in enumerate(segs):
        T = before + count
        k = torch.randn(T, Hkv, D, generator=gen(seed + 3 * i)).to(dtype).float()
        v = torch.randn(T, Hkv, D, generator=gen(seed + 3 * i + 1)).to(dtype).float()
        q = torch.randn(count, Hq, D, generator=gen(seed + 3 * i + 2)).to(dtype).float()
        kvs.append((k, v))
        qs.append(q)
        wants.append(fast_plain_attention(q, k, v, before, window, scale))
    cache, table = make_cache(kvs, page, dtype, seed)
    positions, seg_of_row, info = segments_meta(segs)
    rows = sum(c for _, c in segs)
    # Queries sit in the first columns of a wider qkv buffer, as in the engine.
    qkv = torch.zeros(rows, (Hq + 2 * Hkv) * D, dtype=dtype, device=DEV)
    qkv[:, :Hq * D] = torch.cat(qs).reshape(rows, Hq * D).to(dtype).to(DEV)
    out = torch.full((rows, Hq * D), float("nan"), dtype=dtype, device=DEV)
    st = status()
    kernel(qkv, out, cache, table, positions, seg_of_row, info, segs, page, Hq, Hkv, D, window, scale, st)
    assert st.item() == 0
    got = out.float().cpu().reshape(rows, Hq, D).double()
    want = torch.cat(wants)
    tol = 2e-5 if dtype is torch.float32 else 2e-2
    assert torch.isfinite(got).all()
    assert torch.allclose(got, want, atol=tol, rtol=tol), f"max diff {(got - want).abs().max():.3e}"


def generic_kernel(qkv, out, cache, table, positions, seg_of_row, info, segs, page, Hq, Hkv, D, window, scale, st):
    F().attention_generic(qkv, out, cache, positions, seg_of_row, table, page, Hq, Hkv, D, window, scale, st)


@pytest.mark.parametrize("case", ATTENTION_CASES, ids=[f"case{i}" for i in range(len(ATTENTION_CASES))])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_generic(case, dtype):
    run_attention_case(dtype, generic_kernel, case, seed=10)


def tensor_core_kernels(chunk=None, tcgen05=False):
    shared = {}     # one set of split counters for all calls: each call leaves them zero

    def kernel(qkv, out, cache, table, positions, seg_of_row, info, segs, page, Hq, Hkv, D, window, scale, st):
        group = Hq // Hkv
        small = [i for i, (_, c) in enumerate(segs) if group <= 16 and c * group <= 16]
        large = [i for i in range(len(segs)) if i not in small]
        if small:
            spans = []
            for i in small:
                start, count = segs[i]
                first = max(0, start - window + 1) if window else 0
                spans.append(start + count - first // 64 * 64)
            ck = chunk or 128
            splits = max(-(-s // ck) for s in spans)
            items = torch.tensor(small, dtype=torch.int32, device=DEV)
            counters = shared.setdefault("counters", torch.zeros(256, dtype=torch.int32, device=DEV))
            partial = torch.full((F().attention_decode_scratch_floats(len(small), Hkv, D, splits),), float("nan"),
                                 device=DEV)
            F().attention_decode_bf16(qkv, out, cache, items, len(small), info, table, page, Hq, Hkv, D, window, scale,
                                      ck, splits, partial, st, counters=counters)
            assert int(counters.abs().sum()) == 0, "the split counters were not left at zero"
        if large and tcgen05:
            assert F().attention_prefill_tcgen05_applies(qkv, out, D, page)
            tiles = torch.tensor([(i, t) for i in large for t in range(0, segs[i][1], 128)], dtype=torch.int32, device=DEV)
            # Cold caches: the tiles then arrive late and in another order, which a missing wait would show.
            torch.empty(64 << 20, dtype=torch.int32, device=DEV).zero_()
            F().attention_prefill_tcgen05(qkv, out, cache, tiles, info, table, page, Hq, Hkv, D, window, scale, st)
        elif large:
            tiles = torch.tensor([(i, t) for i in large for t in range(0, segs[i][1], 64)], dtype=torch.int32, device=DEV)
            F().attention_prefill_bf16(qkv, out, cache, tiles, info, table, page, Hq, Hkv, D, window, scale, st)
    return kernel


@pytest.mark.parametrize("case", ATTENTION_CASES, ids=[f"case{i}" for i in range(len(ATTENTION_CASES))])
@pytest.mark.parametrize("chunk", [64, 128, 4096])
def test_attention_tensor_core_kernels(case, chunk):
    if case[2] % 16:
        pytest.skip("head size is no multiple of 16")
    run_attention_case(torch.bfloat16, tensor_core_kernels(chunk), case, seed=20)


TCGEN05_CASES = [
    # Hq, Hkv, D, page, [(context before, new tokens)], window
    (32, 8, 128, 16, [(0, 129), (1536, 64), (63, 2)], 0),
    (16, 8, 128, 64, [(300, 200), (5, 1)], 128),
    (4, 4, 128, 16, [(0, 128)], 0),
    (4, 2, 128, 16, [(0, 64)], 0),
    (6, 2, 64, 8, [(0, 300), (77, 131), (1000, 17)], 0),
    (3, 1, 64, 32, [(130, 270), (0, 5)], 90),
    (8, 2, 128, 128, [(250, 390)], 0),
    (2, 1, 128, 256, [(1000, 700)], 300),
    (10, 5, 64, 16, [(0, 1), (31, 33), (640, 128)], 64),
]


@pytest.mark.parametrize("case", TCGEN05_CASES, ids=[f"case{i}" for i in range(len(TCGEN05_CASES))])
def test_attention_prefill_tcgen05(case):
    run_attention_case(torch.bfloat16, tensor_core_kernels(128, tcgen05=True), case, seed=30)


def test_tensor_core_kernels_refuse_what_they_cannot_do():
    from mini_llm_runtime_b200.ops.native import KernelError
    q = torch.zeros(1, 24 * 3, dtype=torch.bfloat16, device=DEV)
    cache = torch.zeros(2, 2, 1, 16, 24, dtype=torch.bfloat16, device=DEV)
    pos, seg, info = segments_meta([(0, 1)])
    table = torch.zeros(1, 1, dtype=torch.int32, device=DEV)
    with pytest.raises(KernelError, match="head size 24 is not a multiple of 16"):
        F().attention_decode_bf16(q, q[:, :24].clone(), cache, None, 1, info, table, 16, 1, 1, 24, 0, 1.0, 64, 1, None, status())
    with pytest.raises(KernelError, match="head size 24"):
        F().attention_prefill_bf16(q, q[:, :24].clone(), cache, torch.zeros(1, 2, dtype=torch.int32, device=DEV), info,
                                   table, 16, 1, 1, 24, 0, 1.0, status())
    with pytest.raises(KernelError, match="outside"):
        big = torch.zeros(1, 3 * 272, dtype=torch.float32, device=DEV)
        F().attention_generic(big, big[:, :272].clone(), torch.zeros(2, 2, 1, 16, 272, device=DEV), pos, seg, table,
                              16, 1, 1, 272, 0, 1.0, status())


@pytest.mark.parametrize("dtype,kernel", [(torch.float32, generic_kernel), (torch.bfloat16, generic_kernel),
                                          (torch.bfloat16, tensor_core_kernels(128))],
                         ids=["generic-f32", "generic-bf16", "tensor-core"])
def test_one_far_key_among_thousands_decides(dtype, kernel):
    """Random keys give near-uniform attention, which hides a kernel that skips or
    repeats a key.  Here one far key (and one at a page edge) matches the query so
    strongly that the output must be that key's value."""
    Hq, Hkv, D, page = 8, 2, 64, 16
    for before, target in [(3000, 7), (3000, 2048 + 15), (1023, 1008), (4096, 4096)]:
        T = before + 1
        k = torch.randn(T, Hkv, D, generator=gen(0)) * 0.1
        v = torch.randn(T, Hkv, D, generator=gen(1))
        q = torch.randn(1, Hq, D, generator=gen(2)) * 0.1
        direction = torch.randn(D, generator=gen(3))
        direction /= direction.norm()
        k[target, :, :] = direction * 40
        q[0, :, :] = direction * 40
        want = v[target].repeat_interleave(Hq // Hkv, 0)
        cache, table = make_cache([(k, v)], page, dtype, seed=before)
        positions, seg_of_row, info = segments_meta([(before, 1)])
        qkv = torch.zeros(1, (Hq + 2 * Hkv) * D, dtype=dtype, device=DEV)
        qkv[:, :Hq * D] = q.reshape(1, -1).to(dtype).to(DEV)
        out = torch.zeros(1, Hq * D, dtype=dtype, device=DEV)
        kernel(qkv, out, cache, table, positions, seg_of_row, info, [(before, 1)], page, Hq, Hkv, D, 0, 1.0, status())
        got = out.float().cpu().reshape(Hq, D)
        assert torch.allclose(got, want.to(dtype).float(), atol=2e-2), f"context {before}, key {target}"


@pytest.mark.parametrize("dtype,kernel", [(torch.float32, generic_kernel), (torch.bfloat16, tensor_core_kernels(64))],
                         ids=["generic", "tensor-core"])
def test_window_edge_is_exact(dtype, kernel):
    """The key just outside the window would dominate if it were read."""
    Hq, Hkv, D, page, window = 4, 1, 32, 8, 24
    for before in (23, 24, 25, 100, 127, 128):
        T = before + 1
        k = torch.randn(T, Hkv, D, generator=gen(0)) * 0.1
        v = torch.randn(T, Hkv, D, generator=gen(1))
        q = torch.randn(1, Hq, D, generator=gen(2))
        outside = before - window
        if outside >= 0:
            k[outside] = q[0, 0] * 50          # must not be seen
            v[outside] = 1000.0
        want = fast_plain_attention(q, k, v, before, window, 1.0)
        assert want.abs().max() < 100
        cache, table = make_cache([(k, v)], page, dtype)
        positions, seg_of_row, info = segments_meta([(before, 1)])
        qkv = torch.zeros(1, (Hq + 2) * D, dtype=dtype, device=DEV)
        qkv[:, :Hq * D] = q.reshape(1, -1).to(dtype).to(DEV)
        out = torch.zeros(1, Hq * D, dtype=dtype, device=DEV)
        kernel(qkv, out, cache, table, positions, seg_of_row, info, [(before, 1)], page, Hq, Hkv, D, window, 1.0, status())
        tol = 1e-4 if dtype is torch.float32 else 3e-2
        assert torch.allclose(out.float().cpu().reshape(1, Hq, D).double(), want, atol=tol, rtol=tol), before


@pytest.mark.parametrize("page,window", [(16, 0), (64, 0), (8, 1500), (128, 2100)])
def test_prefill_tcgen05_far_keys_and_window_edges(page, window):
    """A portion of 200 tokens after 3000 others.  Some rows look for one far key each (the
    output must be that key's value: a skipped or repeated tile would show); with a window,
    other rows have a key just outside it that would dominate if it were read."""
    Hq, Hkv, D, before, count = 4, 2, 128, 3000, 200
    T = before + count
    dtype = torch.bfloat16
    k = torch.randn(T, Hkv, D, generator=gen(0)) * 0.1
    v = torch.randn(T, Hkv, D, generator=gen(1))
    q = torch.randn(count, Hq, D, generator=gen(2)) * 0.01
    basis = torch.linalg.qr(torch.randn(D, D, generator=gen(3)))[0]
    lowest = before - window + 1 if window else 0           # first key row 0 may read
    targets = {0: lowest, 77: lowest + 77 + 63, 130: before + 64, 199: before + 199, 128: 2048 + 15}
    for n, (row, key) in enumerate(targets.items()):
        k[key] = basis[n] * 40
        q[row] = basis[n] * 40
    hidden = {}
    if window:
        for n, row in enumerate((5, 64, 127, 190)):
            key = before + row - window                     # just outside this row's window
            k[key] = basis[10 + n] * 40
            v[key] = 1000.0
            q[row] = basis[10 + n] * 40
            hidden[row] = key
    want = fast_plain_attention(q, k, v, before, window, 1.0)
    for row, key in targets.items():
        assert torch.allclose(want[row].float(), v[key].repeat_interleave(Hq // Hkv, 0), atol=1e-3)
    assert want.abs().max() < 100
    cache, table = make_cache([(k, v)], page, dtype, seed=page)
    positions, seg_of_row, info = segments_meta([(before, count)])
    qkv = torch.zeros(count, (Hq + 2 * Hkv) * D, dtype=dtype, device=DEV)
    qkv[:, :Hq * D] = q.reshape(count, -1).to(dtype).to(DEV)
    out = torch.zeros(count, Hq * D, dtype=dtype, device=DEV)
    st = status()
    tensor_core_kernels(128, tcgen05=True)(qkv, out, cache, table, positions, seg_of_row, info, [(before, count)], page,
                                           Hq, Hkv, D, window, 1.0, st)
    assert int(st.item()) == 0
    got = out.float().cpu().reshape(count, Hq, D)
    assert torch.isfinite(got).all()
    assert torch.allclose(got.double(), want, atol=3e-2, rtol=3e-2), f"max diff {(got.double() - want).abs().max():.3e}"


# ------------------------------------------------------------------ q/k norm, rotation, cache write
# Few rows take the kernel of one warp per head; many rows in bfloat16 with a head size of 64,
# 128 or 256 take the wide one (several heads per warp), with norm weights of either precision.
@pytest.mark.parametrize("segs", [[(5, 9), (0, 3), (30, 1)], [(5, 29), (0, 3), (30, 1), (60, 21)]], ids=["few-rows", "many-rows"])
@pytest.mark.parametrize("Hq,Hkv,D,page", [(4, 2, 16, 4), (5, 1, 48, 16), (32, 8, 128, 16), (3, 3, 256, 8), (2, 1, 6, 2),
                                           (7, 2, 64, 8), (5, 3, 128, 32)])
@pytest.mark.parametrize("dtype,wdtype", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                          (torch.bfloat16, torch.float32)], ids=["f32", "bf16", "bf16-f32weights"])
def test_qk_norm_rope_cache(Hq, Hkv, D, page, dtype, wdtype, segs):
    from mini_llm_runtime_b200.parts.rotary import rotation_table
    rows = sum(c for _, c in segs)
    theta, eps = 50000.0, 1e-5
    qkv = torch.randn(rows, (Hq + 2 * Hkv) * D, generator=gen(0)).to(dtype)
    wq = (1 + 0.1 * torch.randn(D, generator=gen(1))).to(dtype).to(wdtype)
    wk = (1 + 0.1 * torch.randn(D, generator=gen(2))).to(dtype).to(wdtype)
    positions, seg_of_row, info = segments_meta(segs)
    table_cs = rotation_table(theta, D, 128)
    cos, sin = P.rope_table(positions.tolist(), D, theta, torch.float32)
    assert torch.allclose(table_cs[positions.long().cpu(), :D // 2], cos, atol=1e-6)
    x = qkv.float()
    q = P.qk_norm_rope(x[:, :Hq * D].reshape(rows, Hq, D), wq.float(), eps, cos, sin)
    k = P.qk_norm_rope(x[:, Hq * D:(Hq + Hkv) * D].reshape(rows, Hkv, D), wk.float(), eps, cos, sin)
    v = x[:, (Hq + Hkv) * D:].reshape(rows, Hkv, D)
    # An empty cache with room for every request.
    kvs = [(torch.zeros(s + c, Hkv, D), torch.zeros(s + c, Hkv, D)) for s, c in segs]
    cache, table = make_cache(kvs, page, dtype, seed=4)
    cache.fill_(float("nan"))
    dev = qkv.to(DEV)
    st = status()
    F().qk_norm_rope_cache(dev, Hq, Hkv, D, wq.to(DEV), wk.to(DEV), eps, table_cs.to(DEV), positions, seg_of_row, table,
                           page, cache, True, st)
    assert st.item() == 0
    tol = 1e-5 if dtype is torch.float32 else 2e-2
    got = dev.float().cpu()
    assert torch.allclose(got[:, :Hq * D].reshape(rows, Hq, D), q, atol=tol, rtol=tol)
    assert torch.allclose(got[:, Hq * D:(Hq + Hkv) * D].reshape(rows, Hkv, D), k, atol=tol, rtol=tol)
    assert torch.equal(got[:, (Hq + Hkv) * D:], x[:, (Hq + Hkv) * D:])
    host_cache, host_table = cache.float().cpu(), table.cpu()
    written = torch.zeros(host_cache.shape[0], page, dtype=torch.bool)
    row = 0
    for i, (start, count) in enumerate(segs):
        for p in range(start, start + count):
            page_id, slot = host_table[i, p // page].item(), p % page
            col = torch.arange(D) ^ ((p & 7) << 3) if dtype is torch.bfloat16 and D in (64, 128, 256) else torch.arange(D)
            assert torch.allclose(host_cache[page_id, 0, :, slot][:, col], k[row], atol=tol, rtol=tol)
            assert torch.equal(host_cache[page_id, 1, :, slot][:, col], v[row].to(dtype).float())
            written[page_id, slot] = True
            row += 1
    # Nothing else was touched.
    assert torch.isnan(host_cache[~written[:, None, None, :, None].expand_as(host_cache)]).all()
    # A run that reads another run's cache writes nothing and leaves k alone.
    cache.fill_(float("nan"))
    dev2 = qkv.to(DEV)
    F().qk_norm_rope_cache(dev2, Hq, Hkv, D, wq.to(DEV), wk.to(DEV), eps, table_cs.to(DEV), positions, seg_of_row, table,
                           page, cache, False, st)
    assert torch.isnan(cache).all() and torch.equal(dev2[:, :Hq * D], dev[:, :Hq * D])
    assert torch.equal(dev2[:, Hq * D:].cpu(), qkv[:, Hq * D:])


@pytest.mark.parametrize("Hq,Hkv,D,page,window", [(32, 8, 128, 16, 0), (4, 2, 16, 4, 0), (5, 1, 48, 16, 0), (3, 3, 256, 8, 0), (14, 2, 64, 8, 0),
                                                  (32, 8, 128, 16, 70), (6, 2, 80, 32, 33), (16, 1, 64, 16, 0)])
@pytest.mark.parametrize("norms,rotate,wdtype", [(True, True, torch.bfloat16), (True, True, torch.float32), (False, True, torch.bfloat16),
                                                 (True, False, torch.bfloat16)], ids=["bf16w", "f32w", "no-norm", "no-rotation"])
def test_decode_attention_that_makes_its_own_rows(Hq, Hkv, D, page, window, norms, rotate, wdtype):
    """The split-KV kernel over the raw output of the q/k/v product (it norms, rotates, writes the cache and attends)
    against the row-wise kernel followed by the plain split-KV kernel: the same cache rows and the same attention,
    for decoded tokens and portions of two and three tokens at the start of a sequence, across page and split
    edges, with a window, with and without norm weights and rotation; nothing else of the cache is touched."""
    from mini_llm_runtime_b200.parts.rotary import rotation_table
    group = Hq // Hkv
    most = max(1, 16 // group)
    segs = [(0, 1), (63, min(2, most)), (64, 1), (127, min(3, most)), (200, 1), (15, min(2, most)), (321, 1), (0, min(3, most))]
    rows = sum(c for _, c in segs)
    eps, scale, chunk = 1e-5, D ** -0.5, 64
    qkv = torch.randn(rows, (Hq + 2 * Hkv) * D, generator=gen(0)).to(torch.bfloat16)
    wq = (1 + 0.1 * torch.randn(D, generator=gen(1))).to(torch.bfloat16).to(wdtype).to(DEV) if norms else None
    wk = (1 + 0.1 * torch.randn(D, generator=gen(2))).to(torch.bfloat16).to(wdtype).to(DEV) if norms else None
    table_cs = rotation_table(50000.0, D, 512).to(DEV) if rotate else None
    positions, seg_of_row, info = segments_meta(segs)
    # Earlier tokens of every request in the cache, the step's own positions filled with NaN.
    kvs = []
    for i, (start, count) in enumerate(segs):
        k = torch.randn(start + count, Hkv, D, generator=gen(10 + i))
        v = torch.randn(start + count, Hkv, D, generator=gen(50 + i))
        k[start:], v[start:] = float("nan"), float("nan")
        kvs.append((k, v))
    cache0, table = make_cache(kvs, page, torch.bfloat16, seed=4)
    longest = max(s + c for s, c in segs)
    max_splits = -(-longest // chunk)
    scratch = torch.empty(F().attention_decode_scratch_floats(len(segs), Hkv, D, max_splits), device=DEV)
    st = status()

    cache_a, qkv_a = cache0.clone(), qkv.to(DEV)
    out_a = torch.full((rows, Hq * D), float("nan"), dtype=torch.bfloat16, device=DEV)
    F().qk_norm_rope_cache(qkv_a, Hq, Hkv, D, wq, wk, eps, table_cs, positions, seg_of_row, table, page, cache_a, True, st)
    F().attention_decode_bf16(qkv_a, out_a, cache_a, None, len(segs), info, table, page, Hq, Hkv, D, window, scale, chunk, max_splits,
                              scratch, st)
    cache_b, qkv_b = cache0.clone(), qkv.to(DEV)
    out_b = torch.full((rows, Hq * D), float("nan"), dtype=torch.bfloat16, device=DEV)
    F().attention_decode_fresh_bf16(qkv_b, out_b, cache_b, None, len(segs), info, table, page, Hq, Hkv, D, window, scale, chunk,
                                    max_splits, scratch, wq, wk, eps, table_cs, st)
    assert st.item() == 0
    assert torch.equal(qkv_b.cpu(), qkv)                                   # the product's output is left alone
    a, b = cache_a.float().cpu(), cache_b.float().cpu()
    assert torch.equal(torch.isnan(a), torch.isnan(b)), "the two routes wrote different cache rows"
    assert torch.allclose(torch.nan_to_num(a), torch.nan_to_num(b), atol=2e-2, rtol=1e-2)
    assert torch.equal(a[:, 1], b[:, 1]) or torch.equal(torch.nan_to_num(a[:, 1]), torch.nan_to_num(b[:, 1]))     # values are copied
    assert not torch.isnan(out_b.float()).any()
    assert torch.allclose(out_a.float().cpu(), out_b.float().cpu(), atol=3e-2, rtol=3e-2), (out_a.float() - out_b.float()).abs().max()


def test_qk_kernel_reports_a_page_outside_the_pool():
    pos, seg, info = segments_meta([(0, 2)])
    qkv = torch.zeros(2, 3 * 16, device=DEV)
    cache = torch.zeros(2, 2, 1, 4, 16, device=DEV)
    table = torch.tensor([[5]], dtype=torch.int32, device=DEV)
    st = status()
    F().qk_norm_rope_cache(qkv, 1, 1, 16, None, None, 1.0, None, pos, seg, table, 4, cache, True, st)
    assert st.item() == 2 and cache.abs().sum() == 0


# ------------------------------------------------------------------ sampling
@pytest.mark.parametrize("rows,vocab", [(1, 5), (7, 515), (3, 151936), (64, 4099)])
def test_greedy_and_temperature_sampling(rows, vocab):
    from mini_llm_runtime_b200.sampling.sampler import Sampler
    logits = torch.randn(rows, vocab, generator=gen(0)) * 2
    logits[0, min(3, vocab - 1)] = logits[0, 1] = logits[0].max() + 1          # a tie: the lowest id wins
    st = status()
    sampler = Sampler(torch.device(DEV), st)
    greedy = sampler.sample(logits.to(DEV)).tolist()
    assert greedy == [P.greedy(r) for r in logits] and greedy[0] == 1
    temps = [0.0 if i % 3 == 0 else 0.5 + 0.3 * i for i in range(rows)]
    for seed in range(3):
        us = [P.uniform_for(seed, i, 9) for i in range(rows)]
        got = sampler.sample(logits.to(DEV), temps, us).tolist()
        for i in range(rows):
            if temps[i] == 0:
                assert got[i] == greedy[i]
                continue
            cdf = P.temperature_cdf(logits[i], temps[i])
            lo = cdf[got[i] - 1].item() if got[i] else 0.0
            # The drawn id's interval of the cumulative distribution holds u (up to rounding of the sums).
            assert lo - 1e-6 <= us[i] <= cdf[got[i]].item() + 1e-6, (i, got[i], us[i])
    assert st.item() == 0
    # Edges of the distribution and a non-finite row.
    peaked = torch.full((2, vocab), -50.0)
    peaked[0, vocab - 1] = 50.0
    peaked[1, 0] = 50.0
    assert sampler.sample(peaked.to(DEV), [1.0, 1.0], [0.999999, 0.0]).tolist() == [vocab - 1, 0]
    logits[rows - 1, vocab // 2] = float("nan")
    assert sampler.sample(logits.to(DEV)).tolist()[rows - 1] == -1 and st.item() == 4
