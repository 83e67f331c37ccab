"""Each kernel alone against a plain float64 PyTorch reference of the same
operation, at sizes other than the engine's, in float32 and bfloat16."""
import math
import random

import numpy as np
import pytest
import torch

import plain_qwen3 as P
from gpu_util import pack_meta as pack_step, split_length
from kipp_b200.engine.batch import StepEntry

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def ops():
    from kipp_b200 import kernels
    return kernels


def status():
    return torch.zeros(4, dtype=torch.int32, device=DEV)


def tol(dtype):
    return dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)


# ------------------------------------------------------------------ embedding, norm
@pytest.mark.parametrize("dtype", DTYPES)
def test_embed_gather(dtype):
    g = torch.Generator().manual_seed(0)
    table = torch.randn(301, 72, generator=g).to(dtype).to(DEV)
    ids = torch.tensor([0, 300, 17, 17, 5], dtype=torch.int32, device=DEV)
    out = torch.empty(5, 72, dtype=torch.float32, device=DEV)
    st = status()
    ops().embed_gather(out, table, ids, st)
    assert torch.equal(out.cpu(), table.float().cpu()[ids.cpu().long()])
    assert st.tolist() == [0, 0, 0, 0]


@pytest.mark.parametrize("out_dtype", DTYPES)
@pytest.mark.parametrize("size", [40, 100, 256, 1028, 2560, 4096, 5000])
def test_rmsnorm(size, out_dtype):
    g = torch.Generator().manual_seed(size)
    x = (torch.randn(7, size, generator=g) * 3).to(DEV)
    for w_dtype in DTYPES:
        w = (1 + 0.2 * torch.randn(size, generator=g)).to(w_dtype).to(DEV)
        out = torch.empty(7, size, dtype=out_dtype, device=DEV)
        ops().rmsnorm(out, x, w, 1e-5)
        ref = P.plain_rmsnorm(x.cpu(), w.float().cpu(), 1e-5)
        assert torch.allclose(out.double().cpu(), ref, **tol(out_dtype))
    rows = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEV)
    out = torch.empty(3, size, dtype=out_dtype, device=DEV)
    ops().rmsnorm(out, x, w, 1e-5, rows)
    assert torch.allclose(out.double().cpu(), ref[[6, 0, 3]], **tol(out_dtype))


@pytest.mark.parametrize("size", [24, 200, 320, 1000, 2560, 5120])
def test_rmsnorm_deferred(size):
    """x * weight alone and the sums of squares beside it; the two give the norm."""
    g = torch.Generator().manual_seed(size + 1)
    x = (torch.randn(9, size, generator=g) * 3).to(DEV)
    for w_dtype in DTYPES:
        w = (1 + 0.2 * torch.randn(size, generator=g)).to(w_dtype).to(DEV)
        for out_dtype in DTYPES:
            out = torch.empty(9, size, dtype=out_dtype, device=DEV)
            ssq = torch.full((9,), -1.0, device=DEV)
            ops().rmsnorm_deferred(out, ssq, x, w)
            assert torch.equal(out.cpu(), (x.cpu() * w.float().cpu()).to(out_dtype))       # one rounding
            assert torch.allclose(ssq.double().cpu(), (x.double().cpu() ** 2).sum(-1), rtol=1e-6)
            both = out.double().cpu() / torch.sqrt(ssq.double().cpu()[:, None] / size + 1e-5)
            assert torch.allclose(both, P.plain_rmsnorm(x.cpu(), w.float().cpu(), 1e-5), **tol(out_dtype))
    rows = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEV)
    out = torch.empty(3, size, dtype=torch.bfloat16, device=DEV)
    ssq = torch.zeros(3, device=DEV)
    ops().rmsnorm_deferred(out, ssq, x, w, rows)
    assert torch.equal(out.cpu(), (x.cpu()[[6, 0, 3]] * w.float().cpu()).to(torch.bfloat16))


# ------------------------------------------------------------------ matrix products
def gemm_ref(a, w, epilogue, base):
    p = a.double().cpu() @ w.double().cpu().t()
    if epilogue == "swiglu":
        return P.plain_silu(p[:, 0::2]) * p[:, 1::2]
    return base.double().cpu() + p if epilogue == "add" else p


@pytest.mark.parametrize("epilogue", ["store", "add", "swiglu"])
@pytest.mark.parametrize("shape", [(1, 10, 24), (37, 130, 72), (64, 64, 16), (5, 1000, 136), (130, 66, 200)])
@pytest.mark.parametrize("dtype", DTYPES)
def test_gemm_simt(dtype, shape, epilogue):
    M, N, K = shape
    g = torch.Generator().manual_seed(M + N)
    a = torch.randn(M, K, generator=g).to(dtype).to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.2).to(dtype).to(DEV)
    odt = torch.float32 if epilogue == "add" else dtype
    out = torch.randn(M, N // 2 if epilogue == "swiglu" else N, generator=g).to(odt).to(DEV)
    ref = gemm_ref(a, w, epilogue, out)
    ops().gemm(out, a, w, epilogue, impl="simt")
    assert torch.allclose(out.double().cpu(), ref, **tol(odt))


@pytest.mark.parametrize("epilogue", ["store", "add", "swiglu"])
@pytest.mark.parametrize("shape", [(1, 128, 64), (8, 256, 128), (17, 250, 192), (64, 1000, 136),
                                   (100, 384, 2568), (300, 640, 520), (5, 2560, 1216), (40, 14400, 136),
                                   (100, 14400, 72)])
def test_gemm_tensor_core(shape, epilogue):
    """tcgen05 kernel: integer data must come out exactly (any wrong tile,
    swizzle or split shows), random data within bfloat16 rounding; K splits of
    1, a forced 3 and the cluster maximum 8.  The last two shapes have so many
    features that, left to itself (splits 0), a store or SwiGLU product of 33 to
    511 tokens takes the kernel with the tokens as rows."""
    from kipp_b200.kernels import gemm_bf16
    M, N, K = shape
    g = torch.Generator().manual_seed(M * 7 + N)
    for integer in (True, False):
        for splits in (0, 1, 3, 8):
            if integer:
                a = torch.randint(-3, 4, (M, K), generator=g).to(torch.bfloat16).to(DEV)
                w = torch.randint(-2, 3, (N, K), generator=g).to(torch.bfloat16).to(DEV)
            else:
                a = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
                w = (torch.randn(N, K, generator=g) * 0.1).to(torch.bfloat16).to(DEV)
            odt = torch.float32 if (epilogue == "add" or integer) else torch.bfloat16
            out = torch.randn(M, N // 2 if epilogue == "swiglu" else N, generator=g).to(odt).to(DEV)
            ref = gemm_ref(a, w, epilogue, out)
            gemm_bf16.run("tc", out, a, w, epilogue, M, splits=splits)
            got = out.double().cpu()
            if integer and epilogue != "swiglu":
                assert torch.equal(got, ref.float().double()), (shape, splits)   # one float32 rounding
            else:
                scale = float(ref.abs().max())
                assert float((got - ref).abs().max()) <= (1e-5 if odt == torch.float32 else 1e-2) * scale
    assert gemm_bf16.status_word(torch.device(DEV)).tolist() == [0, 0, 0, 0]


@pytest.mark.parametrize("epilogue", ["store", "add", "swiglu"])
@pytest.mark.parametrize("shape", [(600, 640, 520), (512, 1000, 136), (130, 250, 192), (1100, 2560, 320),
                                   (1024, 384, 4160)])
def test_gemm_tensor_core_tokens_as_rows(shape, epilogue):
    """The orientation used for prompt-sized batches (tokens = MMA rows; a
    thread of the epilogue owns a token and writes vectors, the residual add
    leaves as reducing TMA stores where the output's pitch allows a tensor map,
    in place otherwise), with every feature tile and ragged edges, by one CTA per
    128-token tile and (-1000 - tile) by a pair of CTAs on one MMA per 256-token
    tile; the output also as a slice of a wider buffer; integer data exactly."""
    from kipp_b200.kernels import gemm_bf16
    M, N, K = shape
    g = torch.Generator().manual_seed(M + 3 * N)
    for integer in (True, False):
        for tile_f in (0, -128, -160, -192, -224, -256, -1128, -1160, -1192, -1224, -1256, -1288, -1320):
            if tile_f == 0 and M < 512:
                continue
            if integer:
                a = torch.randint(-3, 4, (M, K), generator=g).to(torch.bfloat16).to(DEV)
                w = torch.randint(-2, 3, (N, K), generator=g).to(torch.bfloat16).to(DEV)
            else:
                a = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
                w = (torch.randn(N, K, generator=g) * 0.1).to(torch.bfloat16).to(DEV)
            odt = torch.float32 if (epilogue == "add" or integer) else torch.bfloat16
            n_out = N // 2 if epilogue == "swiglu" else N
            wide = torch.randn(M + 1, n_out + 8, generator=g).to(odt).to(DEV)
            out = wide[:M, 4:4 + n_out] if tile_f in (-160, -224, -1192) else wide[:M, :n_out].contiguous()
            before = wide.clone()
            ref = gemm_ref(a, w, epilogue, out)
            gemm_bf16.run("tc", out, a, w, epilogue, M, tile_f=tile_f)
            got = out.double().cpu()
            if not out.is_contiguous():                     # nothing beside the slice is touched
                after = wide.clone()
                after[:M, 4:4 + n_out] = before[:M, 4:4 + n_out]
                assert torch.equal(after, before), (shape, tile_f)
            if integer and epilogue != "swiglu":
                assert torch.equal(got, ref.float().double()), (shape, tile_f)
            else:
                scale = float(ref.abs().max())
                assert float((got - ref).abs().max()) <= (1e-5 if odt == torch.float32 else 1e-2) * scale
    assert gemm_bf16.status_word(torch.device(DEV)).tolist() == [0, 0, 0, 0]


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_gemm_tensor_core_left_to_choose_its_kernel(seed):
    """Shapes drawn around every boundary of the choice of kernel and tile (tokens 1 to
    2,100, features 8 to 20,000, K 8 to 4,104, ragged in every direction), the three
    epilogues, both output types, with and without the row factors of a deferred norm:
    whatever kernel the launcher takes, the product matches the plain one."""
    from kipp_b200.kernels import gemm_bf16
    rng = random.Random(seed)
    for trial in range(40):
        M = rng.choice([1, 3, 8, 16, 17, 31, 32, 33, 40, 64, 65, 100, 128, 200, 256, 300, 400, 511, 512, 513, 700,
                        1000, 1023, 1024, 1025, 1300, 1536, 2048, 2100])
        N = rng.choice([8, 24, 128, 136, 256, 1000, 2560, 2568, 4096, 6144, 9000, 14400, 19456, 20000])
        K = rng.choice([8, 64, 72, 128, 520, 1024, 2560, 4104])
        epilogue = rng.choice(["store", "add", "swiglu"])
        g = torch.Generator(device=DEV).manual_seed(1000 * seed + trial)
        a = torch.randn(M, K, generator=g, device=DEV).to(torch.bfloat16)
        w = (torch.randn(N, K, generator=g, device=DEV) * 0.1).to(torch.bfloat16)
        odt = torch.float32 if epilogue == "add" else rng.choice([torch.float32, torch.bfloat16])
        out = torch.randn(M, N // 2 if epilogue == "swiglu" else N, generator=g, device=DEV).to(odt)
        prod = a.double() @ w.double().t()
        fold = None
        if epilogue != "add" and rng.random() < 0.4:
            ssq = torch.rand(M, 5, generator=g, device=DEV) * 30 + 1
            fold = gemm_bf16.fold_scale(ssq, 77, 1e-5)
            prod = prod * torch.rsqrt(ssq.double().sum(1) / 77 + 1e-5)[:, None]
        if epilogue == "add":
            ref = out.double() + prod
        elif epilogue == "swiglu":
            ref = prod[:, 0::2] / (1 + torch.exp(-prod[:, 0::2])) * prod[:, 1::2]
        else:
            ref = prod
        gemm_bf16.run("tc", out, a, w, epilogue, M, fold=fold)
        scale = float(ref.abs().max()) + 1e-9
        err = float((out.double() - ref).abs().max()) / scale
        assert err <= (2e-5 if odt == torch.float32 else 1e-2), (M, N, K, epilogue, odt, fold is not None, err)
    assert gemm_bf16.status_word(torch.device(DEV)).tolist() == [0, 0, 0, 0]


@pytest.mark.parametrize("wdtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(1, 128, 64), (8, 256, 128), (17, 224, 192), (64, 992, 136), (100, 384, 2568),
                                   (300, 640, 520), (5, 2560, 1216)])
def test_gemm_folds_the_norm_around_it(shape, wdtype):
    """The few-token kernel with an RMSNorm folded in: the residual add also leaves
    bf16(new residual x norm weight) and the sums of squares of the new residual per
    32 features; a store or SwiGLU product scales row t by 1 / sqrt(sum / n + eps).
    Integer data exactly; every K split, the cluster's reduction included."""
    from kipp_b200.kernels import gemm_bf16
    M, N, K = shape
    g = torch.Generator().manual_seed(M * 5 + N)
    for splits in (0, 1, 3, 8):
        a = torch.randint(-3, 4, (M, K), generator=g).to(torch.bfloat16).to(DEV)
        w = torch.randint(-2, 3, (N, K), generator=g).to(torch.bfloat16).to(DEV)
        base = torch.randint(-8, 9, (M, N), generator=g).float().to(DEV)
        nw = (torch.randint(1, 5, (N,), generator=g).float() * 0.25).to(wdtype).to(DEV)
        out = base.clone()
        xn = torch.full((M, N + 8), 7.0, dtype=torch.bfloat16, device=DEV)
        ssq = torch.full((M, N // 32), -1.0, device=DEV)
        gemm_bf16.run("tc", out, a, w, "add", M, splits=splits, fold=gemm_bf16.fold_emit(nw, xn, ssq))
        ref = gemm_ref(a, w, "add", base).float()
        assert torch.equal(out.cpu(), ref), (shape, splits)
        assert torch.equal(xn[:, :N].float().cpu(), (ref * nw.float().cpu()).to(torch.bfloat16).float())
        assert torch.all(xn[:, N:] == 7.0)
        assert torch.equal(ssq.cpu(), (ref * ref).view(M, N // 32, 32).sum(-1))
        # the consumer: rows scaled by the factor that the sums give
        eps = 1e-3
        rstd = 1.0 / torch.sqrt(ssq.double().cpu().sum(-1, keepdim=True) / N + eps)
        for epilogue in ("store", "swiglu"):
            n_out = N // 2 if epilogue == "swiglu" else N
            got = torch.zeros(M, n_out, device=DEV)
            gemm_bf16.run("tc", got, a, w, epilogue, M, splits=splits, fold=gemm_bf16.fold_scale(ssq, N, eps))
            p = (a.double().cpu() @ w.double().cpu().t()) * rstd
            want = P.plain_silu(p[:, 0::2]) * p[:, 1::2] if epilogue == "swiglu" else p
            assert float((got.double().cpu() - want).abs().max()) <= 2e-6 * max(1.0, float(want.abs().max()))
        # ... and so do the kernels of prompt-sized batches (forced here), which cannot emit
        for tile_f in (-128, -1160):
            for epilogue in ("store", "swiglu"):
                n_out = N // 2 if epilogue == "swiglu" else N
                got = torch.zeros(M, n_out, device=DEV)
                gemm_bf16.run("tc", got, a, w, epilogue, M, tile_f=tile_f, fold=gemm_bf16.fold_scale(ssq, N, eps))
                p = (a.double().cpu() @ w.double().cpu().t()) * rstd
                want = P.plain_silu(p[:, 0::2]) * p[:, 1::2] if epilogue == "swiglu" else p
                assert float((got.double().cpu() - want).abs().max()) <= 2e-6 * max(1.0, float(want.abs().max()))
            with pytest.raises(Exception):
                gemm_bf16.run("tc", out, a, w, "add", M, tile_f=tile_f, fold=gemm_bf16.fold_emit(nw, xn, ssq))
    assert gemm_bf16.status_word(torch.device(DEV)).tolist() == [0, 0, 0, 0]


def test_gemm_refuses_what_it_cannot_take():
    from kipp_b200.kernels import KernelError, gemm_bf16
    a = torch.zeros(4, 20, dtype=torch.bfloat16, device=DEV)          # K = 20: row pitch not 16-byte
    w = torch.zeros(8, 20, dtype=torch.bfloat16, device=DEV)
    out = torch.zeros(4, 8, dtype=torch.bfloat16, device=DEV)
    assert not gemm_bf16.tc_ok(a, w)
    with pytest.raises(KernelError):
        gemm_bf16.run("tc", out, a, w, "store", 4)
    ops().gemm(out, a, w, "store")                                     # the default path takes it (CUDA cores)
    with pytest.raises(KernelError):
        ops().gemm(out, a.cpu(), w, "store")


# ------------------------------------------------------------------ norm + rotation + cache write
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", [dict(D=16, nq=4, nkv=2, rot=16, norm=True, page=4),
                                  dict(D=80, nq=3, nkv=3, rot=80, norm=True, page=16),
                                  dict(D=128, nq=8, nkv=1, rot=128, norm=False, page=8),
                                  dict(D=64, nq=2, nkv=2, rot=32, norm=True, page=16),
                                  dict(D=256, nq=2, nkv=1, rot=0, norm=True, page=32),
                                  dict(D=128, nq=9, nkv=3, rot=128, norm=True, page=16, long=290),
                                  dict(D=48, nq=5, nkv=5, rot=16, norm=True, page=8, long=260),
                                  dict(D=64, nq=5, nkv=2, rot=64, norm=True, page=8, long=130, w16=True),
                                  dict(D=256, nq=3, nkv=2, rot=256, norm=True, page=16, long=70, w16=True)])
def test_qk_norm_rope_write(case, dtype):
    """Cases with `long` have many tokens: several heads per warp.  In bfloat16
    the head sizes 64, 128 and 256 with a full or no rotation take the
    16-byte-vector kernel (head counts that leave a warp's last heads empty or
    put a key and a value head into one warp); `w16` has the norm weights in
    bfloat16 as checkpoints store them."""
    D, nq, nkv, rot, page = case["D"], case["nq"], case["nkv"], case["rot"], case["page"]
    g = torch.Generator().manual_seed(D)
    n_long = case.get("long", 19)
    entries = [StepEntry("a", [0] * 5, []), StepEntry("b", [0] * 1, []), StepEntry("c", [0] * n_long, [])]
    starts = [13, 40, 0]
    width = -(-max(45, n_long + 1) // page)
    n_pages = 3 * width
    perm = torch.randperm(n_pages, generator=g).int().numpy().reshape(3, width)
    meta = pack_step(entries, starts, [0, 1, 2], [perm.astype(np.int32)], torch.device(DEV))
    T = meta.tokens
    qkv = torch.randn(T, (nq + 2 * nkv) * D, generator=g).to(dtype).to(DEV)
    wdt = torch.bfloat16 if case.get("w16") else torch.float32
    qw = (1 + 0.2 * torch.randn(D, generator=g)).to(wdt).to(DEV) if case["norm"] else None
    kw = (1 + 0.2 * torch.randn(D, generator=g)).to(wdt).to(DEV) if case["norm"] else None
    theta = 10000.0
    inv = None
    if rot:
        i = torch.arange(rot // 2, dtype=torch.float32)
        inv = torch.pow(torch.tensor(theta, dtype=torch.float64), (-(2.0 * i) / rot).double()).float().to(DEV)
    q_out = torch.zeros(T, nq, D, dtype=dtype, device=DEV)
    kp = torch.zeros(n_pages, nkv, page, D, dtype=dtype, device=DEV)
    vp = torch.zeros_like(kp)
    st = status()
    ops().qk_norm_rope_write(qkv, q_out, kp, vp, qw, kw, 1e-6, inv, rot, meta.positions,
                             meta.entry_of_token, meta.block_tables[0], page, T, nq, nkv, D, True, st)
    assert st.tolist() == [0, 0, 0, 0]
    x = qkv.double().cpu().reshape(T, nq + 2 * nkv, D)
    pos = meta.positions.cpu().tolist()

    def transform(h, w):
        if w is not None:
            h = P.plain_rmsnorm(h, w.cpu(), 1e-6)
        if rot:
            h = torch.cat([P.plain_rope(h[..., :rot].float(), pos, theta), h[..., rot:].double()], -1)
        return h
    q_ref, k_ref, v_ref = transform(x[:, :nq], qw), transform(x[:, nq:nq + nkv], kw), x[:, nq + nkv:]
    assert torch.allclose(q_out.double().cpu(), q_ref, **tol(dtype))
    ent = meta.entry_of_token.cpu().tolist()
    written = torch.zeros(n_pages, page, dtype=torch.bool)
    for t in range(T):
        pg, sl = int(perm[ent[t], pos[t] // page]), pos[t] % page
        assert torch.allclose(kp[pg, :, sl].double().cpu(), k_ref[t], **tol(dtype)), t
        assert torch.allclose(vp[pg, :, sl].double().cpu(), v_ref[t], **tol(dtype)), t
        written[pg, sl] = True
    assert float(kp.float().abs().sum(dim=(1, 3)).cpu()[~written].sum()) == 0.0    # nothing else touched
    # a run that reads another run's cache writes nothing
    kp2 = torch.zeros_like(kp)
    ops().qk_norm_rope_write(qkv, q_out, kp2, kp2, qw, kw, 1e-6, inv, rot, meta.positions,
                             meta.entry_of_token, meta.block_tables[0], page, T, nq, nkv, D, False, st)
    assert float(kp2.float().abs().sum()) == 0.0


@pytest.mark.parametrize("case", [
    dict(T=1024, nq=4, nkv=2, K=192, norm=True, rot=True, page=16, scaled=False),
    dict(T=1300, nq=5, nkv=1, K=320, norm=True, rot=True, page=8, scaled=True, w16=True),   # 7 heads: half a tile empty
    dict(T=1100, nq=2, nkv=2, K=128, norm=False, rot=True, page=64, scaled=False),
    dict(T=1030, nq=3, nkv=3, K=256, norm=True, rot=False, page=32, scaled=True),
])
def test_projection_hands_its_heads_to_attention(case):
    """The q/k/v projection of a prompt-sized step with per-head norm, rotation and
    the cache write in its epilogue: the same bits as the stored product followed
    by `qk_norm_rope_write`, with and without the row factors of a deferred norm;
    two requests in the step, permuted pages, a token count that fills no tile."""
    from kipp_b200.kernels import gemm_bf16
    D = 128
    T, nq, nkv, K, page = case["T"], case["nq"], case["nkv"], case["K"], case["page"]
    assert gemm_bf16.heads_ok(T, D, D if case["rot"] else 0) and not gemm_bf16.heads_ok(1023, D, D)
    assert not gemm_bf16.heads_ok(T, 64, 64) and not gemm_bf16.heads_ok(T, D, 64)
    g = torch.Generator().manual_seed(T + nq)
    n_a = 37
    entries = [StepEntry("a", [0] * n_a, []), StepEntry("b", [0] * (T - n_a), [])]
    starts = [29, 3]
    width = -(-(T + 40) // page)
    perm = torch.randperm(2 * width, generator=g).int().numpy().reshape(2, width)
    meta = pack_step(entries, starts, [0, 1], [perm.astype(np.int32)], torch.device(DEV))
    a = torch.randn(T, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn((nq + 2 * nkv) * D, K, generator=g) / math.sqrt(K)).to(torch.bfloat16).to(DEV)
    wdt = torch.bfloat16 if case.get("w16") else torch.float32
    qw = (1 + 0.2 * torch.randn(D, generator=g)).to(wdt).to(DEV) if case["norm"] else None
    kw = (1 + 0.2 * torch.randn(D, generator=g)).to(wdt).to(DEV) if case["norm"] else None
    inv = None
    cos_sin = by_pair = None
    if case["rot"]:
        i = torch.arange(D // 2, dtype=torch.float32)
        inv = torch.pow(torch.tensor(10000.0, dtype=torch.float64), (-(2.0 * i) / D).double()).float().to(DEV)
        cos_sin = ops().rope_table(meta.positions, inv, T)
        by_pair = ops().rope_table(meta.positions, inv, T, by_pair=True)
        assert torch.equal(by_pair.transpose(0, 1), cos_sin)
    fold = None
    if case["scaled"]:
        ssq = (torch.rand(T, 3, generator=g) * 40 + 1).to(DEV)
        fold = gemm_bf16.fold_scale(ssq, 96, 1e-5)
    st = status()

    def pools():
        return (torch.zeros(T, nq, D, dtype=torch.bfloat16, device=DEV),
                torch.zeros(2 * width, nkv, page, D, dtype=torch.bfloat16, device=DEV),
                torch.zeros(2 * width, nkv, page, D, dtype=torch.bfloat16, device=DEV))
    q1, k1, v1 = pools()
    qkv = torch.empty(T, (nq + 2 * nkv) * D, dtype=torch.bfloat16, device=DEV)
    gemm_bf16.run("tc", qkv, a, w, "store", T, fold=fold, status=st)
    ops().qk_norm_rope_write(qkv, q1, k1, v1, qw, kw, 1e-6, inv, D if case["rot"] else 0, meta.positions,
                             meta.entry_of_token, meta.block_tables[0], page, T, nq, nkv, D, True, st,
                             cos_sin=cos_sin)
    q2, k2, v2 = pools()
    gemm_bf16.run_heads(a, w, q2, k2, v2, qw, kw, 1e-6, by_pair, meta.positions, meta.entry_of_token,
                        meta.block_tables[0], nq, nkv, status=st, fold=fold)
    torch.cuda.synchronize()
    assert st.tolist() == [0, 0, 0, 0]
    assert float(q1.float().abs().sum()) > 0 and float(k1.float().abs().sum()) > 0
    assert torch.equal(q1, q2) and torch.equal(k1, k2) and torch.equal(v1, v2)
    # a run that reads another run's cache writes nothing
    q3, k3, v3 = pools()
    gemm_bf16.run_heads(a, w, q3, k3, v3, qw, kw, 1e-6, by_pair, meta.positions, meta.entry_of_token,
                        meta.block_tables[0], nq, nkv, write_cache=False, status=st, fold=fold)
    assert torch.equal(q1, q3) and float(k3.float().abs().sum()) == 0.0 and float(v3.float().abs().sum()) == 0.0
    # an unmapped page is refused through the status word and nothing is written there
    table = meta.block_tables[0].clone()
    table[1, 5] = -1
    q4, k4, v4 = pools()
    gemm_bf16.run_heads(a, w, q4, k4, v4, qw, kw, 1e-6, by_pair, meta.positions, meta.entry_of_token, table,
                        nq, nkv, status=st, fold=fold)
    assert st.tolist() == [2, 0, 0, 0]
    st.zero_()
    untouched = int(perm[1, 5])
    assert float(k4[untouched].float().abs().sum()) == 0.0
    others = [i for i in range(2 * width) if i != untouched]
    assert torch.equal(k4[others], k1[others]) and torch.equal(q4, q1)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("D", [48, 128])
def test_no_infinity_or_nan_reaches_the_cache(D, dtype):
    """A page goes from one request to the next as it is, and kernels that read whole
    tiles multiply masked keys and values by zero: so a key or value that is not
    finite (an overflow in one request) is stored as 0, in both kernels that write
    the cache."""
    nq, nkv, page, T = 4, 2, 8, 5
    g = torch.Generator().manual_seed(D)
    entries = [StepEntry("a", [0] * T, [])]
    meta = pack_step(entries, [0], [0], [np.arange(2, dtype=np.int32).reshape(1, 2)], torch.device(DEV))
    qkv = torch.randn(T, (nq + 2 * nkv) * D, generator=g).to(dtype)
    k0, v0 = nq * D, (nq + nkv) * D
    qkv[1, k0 + 3] = float("inf")              # a key element; with the norm the whole head turns NaN
    qkv[2, v0 + 5] = float("nan")
    qkv[3, v0 + D + 1] = float("-inf")
    qkv = qkv.to(DEV)
    kw = torch.ones(D, device=DEV)
    kp = torch.zeros(2, nkv, page, D, dtype=dtype, device=DEV)
    vp = torch.zeros_like(kp)
    q_out = torch.zeros(T, nq, D, dtype=dtype, device=DEV)
    st = status()
    ops().qk_norm_rope_write(qkv, q_out, kp, vp, kw, kw, 1e-6, None, 0, meta.positions, meta.entry_of_token,
                             meta.block_tables[0], page, T, nq, nkv, D, True, st)
    torch.cuda.synchronize()
    assert torch.isfinite(kp.float()).all() and torch.isfinite(vp.float()).all()
    assert float(kp[0, 0, 1].float().abs().sum()) == 0.0           # the poisoned key head became zeros
    assert float(vp[0, 0, 2, 5]) == 0.0 and float(vp[0, 1, 3, 1]) == 0.0
    assert float(vp[0, 0, 2, 4]) == float(qkv[2, v0 + 4])          # its finite neighbours are kept
    assert float(kp[0, 1, 1].float().abs().sum()) > 0              # and the other key head of that token


# ------------------------------------------------------------------ attention
def attention_case(seed, D, nq, nkv, page, layout, dtype, width=None, order="permuted"):
    """layout: list of (cached tokens, new tokens).  Random pages in a permuted
    pool (order "consecutive": page ids in a row, as a request gets them from a
    fresh pool; "runs": rows of 1 to 9 consecutive ids, in shuffled order);
    returns everything the kernels and the reference need."""
    g = torch.Generator().manual_seed(seed)
    entries = [StepEntry(i, [0] * n, []) for i, (_, n) in enumerate(layout)]
    starts = [c for c, _ in layout]
    need = [-(-(c + n) // page) for c, n in layout]
    width = width or max(need)
    n_pages = sum(need) + 3
    if order == "consecutive":
        perm = list(range(2, n_pages))
    elif order == "runs":
        runs, at = [], 0
        while at < n_pages:
            k = int(torch.randint(1, 10, (1,), generator=g))
            runs.append(list(range(at, min(at + k, n_pages))))
            at += k
        perm = [x for i in torch.randperm(len(runs), generator=g).tolist() for x in runs[i]]
    else:
        perm = torch.randperm(n_pages, generator=g).int().tolist()
    table = np.full((len(layout), width), -1, dtype=np.int32)
    at = 0
    for i, k in enumerate(need):
        table[i, :k] = perm[at:at + k]
        at += k
    meta = pack_step(entries, starts, list(range(len(layout))), [table], torch.device(DEV))
    q = torch.randn(meta.tokens, nq, D, generator=g).to(dtype).to(DEV)
    kp = torch.randn(n_pages, nkv, page, D, generator=g).to(dtype).to(DEV)
    vp = torch.randn(n_pages, nkv, page, D, generator=g).to(dtype).to(DEV)
    return meta, table, q, kp, vp


def attention_ref(meta, table, q, kp, vp, layout, page, window, scale):
    T, nq, D = q.shape
    nkv = kp.shape[1]
    out = torch.zeros(T, nq, D, dtype=torch.float64)
    qc, kc, vc = q.double().cpu(), kp.double().cpu(), vp.double().cpu()
    t = 0
    for e, (ctx, n) in enumerate(layout):
        total = ctx + n
        pages = torch.tensor(table[e, :-(-total // page)].tolist())
        keys = kc[pages].permute(0, 2, 1, 3).reshape(-1, nkv, D)[:total]
        vals = vc[pages].permute(0, 2, 1, 3).reshape(-1, nkv, D)[:total]
        for i in range(n):
            pos = ctx + i
            lo = 0 if not window else max(0, pos - window + 1)
            for h in range(nq):
                gk = h // (nq // nkv)
                s = (keys[lo:pos + 1, gk] @ qc[t, h]) * scale
                out[t, h] = P.plain_softmax(s) @ vals[lo:pos + 1, gk]
            t += 1
    return out


LAYOUTS = [[(0, 70), (130, 1), (5, 2), (63, 66), (300, 1)],
           [(0, 1), (1, 1), (15, 1), (16, 1), (255, 1), (256, 1), (257, 1), (700, 1)],
           [(0, 200)], [(100, 3), (0, 64), (64, 64), (127, 2)]]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [None, 37])
@pytest.mark.parametrize("shape", [dict(D=16, nq=4, nkv=2, page=16), dict(D=48, nq=6, nkv=3, page=8),
                                   dict(D=128, nq=8, nkv=1, page=4), dict(D=256, nq=2, nkv=2, page=32)])
def test_attention_simt(shape, window, dtype):
    D, nq, nkv, page = shape["D"], shape["nq"], shape["nkv"], shape["page"]
    for li, layout in enumerate(LAYOUTS[:2] + LAYOUTS[3:]):
        meta, table, q, kp, vp = attention_case(li, D, nq, nkv, page, layout, dtype)
        out = torch.zeros_like(q)
        st = status()
        ops().attention(out, q, kp, vp, meta, meta.block_tables[0], page, nq, nkv, D, 1 / math.sqrt(D),
                        window, st, impl="simt")
        ref = attention_ref(meta, table, q, kp, vp, layout, page, window, 1 / math.sqrt(D))
        assert st.tolist() == [0, 0, 0, 0]
        assert torch.allclose(out.double().cpu(), ref, **tol(dtype)), (shape, li)


@pytest.mark.parametrize("window", [None, 37, 300])
@pytest.mark.parametrize("shape", [dict(D=64, nq=4, nkv=2, page=16), dict(D=128, nq=8, nkv=2, page=16),
                                   dict(D=128, nq=16, nkv=1, page=8), dict(D=64, nq=3, nkv=3, page=32),
                                   dict(D=128, nq=40, nkv=2, page=16), dict(D=128, nq=4, nkv=2, page=64),
                                   dict(D=64, nq=2, nkv=1, page=128), dict(D=128, nq=2, nkv=2, page=4)])
def test_attention_tensor_core(shape, window):
    """Prompt portions and single decoded tokens through the tensor-core kernels:
    portions of 64 tokens and more through tcgen05, shorter ones and decoded
    tokens through mma.sync (a group of 20 > 16 and a page of 4 slots go through
    the mma.sync portion kernel throughout; pages of 64 and 128 slots hold a whole
    key tile); then the same with tcgen05 off."""
    from kipp_b200.kernels import attention_bf16
    D, nq, nkv, page = shape["D"], shape["nq"], shape["nkv"], shape["page"]
    assert attention_bf16.supported(D, nq, nkv)
    for li, layout in enumerate(LAYOUTS):
        meta, table, q, kp, vp = attention_case(10 + li, D, nq, nkv, page, layout, torch.bfloat16)
        out = torch.full_like(q, 9.0)
        st = status()
        # whatever lies in the split-K scratch must not matter: a split wholly behind a
        # window writes no partial output, and 0 x NaN would be NaN
        attention_bf16.decode_scratch(torch.device(DEV), meta.tokens, nq, D).fill_(float("nan"))
        ops().attention(out, q, kp, vp, meta, meta.block_tables[0], page, nq, nkv, D, 1 / math.sqrt(D),
                        window, st, impl="mma")
        ref = attention_ref(meta, table, q, kp, vp, layout, page, window, 1 / math.sqrt(D))
        assert torch.allclose(out.double().cpu(), ref, rtol=2e-2, atol=2e-2), (shape, li, window)
        assert st.tolist() == [0, 0, 0, 0]
        # the decoded tokens cut into splits of a given length instead of dealt out as a stream
        out1 = torch.full_like(q, 9.0)
        attention_bf16.run("mma", out1, q, kp, vp, meta, meta.block_tables[0], page, nq, nkv, D, 1 / math.sqrt(D),
                           window, st, stream=False)
        assert torch.allclose(out1.double().cpu(), ref, rtol=2e-2, atol=2e-2), (shape, li, window)
        attention_bf16.PREFILL_TC = False
        try:
            out2 = torch.full_like(q, 9.0)
            ops().attention(out2, q, kp, vp, meta, meta.block_tables[0], page, nq, nkv, D, 1 / math.sqrt(D),
                            window, st, impl="mma")
        finally:
            attention_bf16.PREFILL_TC = True
        assert torch.allclose(out2.double().cpu(), ref, rtol=2e-2, atol=2e-2), (shape, li, window)


@pytest.mark.parametrize("order", ["consecutive", "runs"])
@pytest.mark.parametrize("page", [8, 16, 32])
@pytest.mark.parametrize("D", [64, 128])
def test_attention_pages_in_a_row(D, page, order):
    """Pages that follow one another in the pool (what a request gets from a fresh
    pool) are fetched as whole key tiles by the prompt kernel, pages in any other
    order one by one: both in one launch, rows of consecutive pages that start and
    end anywhere in a tile."""
    nq, nkv = 4, 2
    for window in (None, 150):
        for li, layout in enumerate([[(0, 700)], [(300, 150), (0, 64), (77, 513)], [(64, 200), (1000, 129)]]):
            meta, table, q, kp, vp = attention_case(40 + li, D, nq, nkv, page, layout, torch.bfloat16, order=order)
            out = torch.full_like(q, 9.0)
            st = status()
            ops().attention(out, q, kp, vp, meta, meta.block_tables[0], page, nq, nkv, D, 1 / math.sqrt(D),
                            window, st, impl="mma")
            ref = attention_ref(meta, table, q, kp, vp, layout, page, window, 1 / math.sqrt(D))
            assert st.tolist() == [0, 0, 0, 0]
            assert torch.allclose(out.double().cpu(), ref, rtol=2e-2, atol=2e-2), (D, page, order, li, window)


@pytest.mark.parametrize("impl,dtype", [("simt", torch.float32), ("simt", torch.bfloat16),
                                        ("mma", torch.bfloat16)])
def test_attention_finds_one_far_key(impl, dtype):
    """Random data would hide a wrong key among hundreds: here each query's
    score is large for exactly one chosen key (the first key, page edges, the
    window's edge, the token itself) and the values name their position."""
    D, nq, nkv, page, window = 128, 4, 2, 16, 100      # D > the longest portion: key directions stay unique
    ctx, n = 419, 5                                  # a portion of 5 tokens, one decoded token, a portion of 70
    for layout in ([(ctx, n)], [(ctx + n - 1, 1)], [(ctx, 70)]):
        meta, table, q, kp, vp = attention_case(3, D, nq, nkv, page, layout, dtype)
        total = layout[0][0] + layout[0][1]
        kp.zero_(); vp.zero_(); q.zero_()
        pages = table[0]
        for pos in range(total):                     # key at pos: e_{pos % D} scaled; value: its position
            kp[pages[pos // page], :, pos % page, pos % D] = 1.0
            vp[pages[pos // page], :, pos % page, 0] = float(pos % 256)
            vp[pages[pos // page], :, pos % page, 1] = float(pos // 256)
        first = layout[0][0]                          # position of the first query
        for win, targets in ((None, [0, 15, 16, 255, 256, first - 65, first - 1, "self"]),
                             (window, ["edge", "edge+1", "mid", "self"])):
            for target in targets:
                q.zero_()
                want = []
                for i in range(layout[0][1]):
                    pos = layout[0][0] + i
                    j = {"self": pos, "edge": pos - window + 1, "edge+1": pos - window + 2,
                         "mid": pos - window // 2}.get(target, target)
                    q[i, :, j % D] = 60.0
                    want.append(j)
                # keys j + k * D point the same way as key j: the wanted key alone is twice as long
                for i, j in enumerate(want):
                    kp[pages[j // page], :, j % page, j % D] = 2.0
                out = torch.zeros_like(q)
                ops().attention(out, q, kp, vp, meta, meta.block_tables[0], page, nq, nkv, D, 1.0, win,
                                status(), impl=impl)
                got = out.float().cpu()
                for i, j in enumerate(want):
                    pos_read = got[i, :, 0] + 256 * got[i, :, 1]
                    assert torch.allclose(pos_read, torch.full((nq,), float(j)), atol=0.6), (target, i, j, pos_read)
                for j in want:
                    kp[pages[j // page], :, j % page, j % D] = 1.0
        # a key just outside the window must NOT be seen even when it is the strongest
        q.zero_()
        pos = layout[0][0] + layout[0][1] - 1
        j = pos - window                               # one before the window's first key
        q[-1, :, j % D] = 60.0
        kp[pages[j // page], :, j % page, j % D] = 4.0
        out = torch.zeros_like(q)
        ops().attention(out, q, kp, vp, meta, meta.block_tables[0], page, nq, nkv, D, 1.0, window, status(),
                        impl=impl)
        got = out.float().cpu()[-1]
        assert (got[:, 0] + 256 * got[:, 1] - float(j)).abs().min() > 1.0
        kp[pages[j // page], :, j % page, j % D] = 1.0


@pytest.mark.parametrize("rate", [0.02, 0.07, 0.3, -0.07])
def test_attention_scores_that_climb(rate):
    """Scores that rise (or fall) steadily with the key's position: the running
    maximum of the prompt kernel drifts by a few units per key tile, so tiles are
    added under a maximum that is not their own before the output is rescaled;
    with random scores the maximum settles in the first tiles and this path sleeps."""
    D, nq, nkv, page = 128, 4, 2, 16
    for layout in ([(0, 700)], [(300, 150), (0, 64)]):
        meta, table, q, kp, vp = attention_case(21, D, nq, nkv, page, layout, torch.bfloat16)
        kp.mul_(0.1)
        q.mul_(0.1)
        q[:, :, 5] = 1.0
        for r, (ctx, n) in enumerate(layout):
            for pos in range(ctx + n):
                kp[table[r][pos // page], :, pos % page, 5] = rate * pos      # score = rate * pos in natural-log units
        out = torch.zeros_like(q)
        st = status()
        ops().attention(out, q, kp, vp, meta, meta.block_tables[0], page, nq, nkv, D, 1.0, None, st, impl="mma")
        ref = attention_ref(meta, table, q, kp, vp, layout, page, None, 1.0)
        assert st.tolist() == [0, 0, 0, 0]
        assert torch.allclose(out.double().cpu(), ref, rtol=2e-2, atol=2e-2), (rate, layout)


# ------------------------------------------------------------------ sampling
def test_burst_advance_moves_a_step_on():
    """The kernels between two greedy steps of a burst: tokens handed over and put into
    the ring row the counter names, positions and cached lengths + 1; then the keys per
    decode-attention split of every token, chosen as the host chooses them for the new
    lengths (for the whole step, or from each token's own context)."""
    from kipp_b200.kernels import attention_bf16, sampling
    g = torch.Generator().manual_seed(5)
    for n, longest in ((1, 100), (1, 2047), (3, 5000), (8, 8190), (8, 127), (64, 2047), (64, 40_000), (130, 700)):
        lens = torch.randint(1, longest + 1, (n,), generator=g).int()
        lens[int(torch.randint(0, n, (1,), generator=g))] = longest
        dev = lambda t: t.clone().to(DEV)
        tokens, positions, context = dev(torch.zeros(n).int()), dev(lens), dev(lens)
        counter = dev(torch.tensor([2]).int())
        nxt = torch.randint(0, 50_000, (n,), generator=g).int()
        ring = torch.full((4, n), -7, dtype=torch.int32, device=DEV)
        sampling.burst_advance(tokens, positions, context, dev(nxt), ring, counter)
        assert tokens.cpu().tolist() == nxt.tolist()
        assert positions.cpu().tolist() == (lens + 1).tolist() == context.cpu().tolist()
        assert int(counter) == 3 and ring[2].cpu().tolist() == nxt.tolist()
        assert ring[[0, 1, 3]].eq(-7).all()
        # the next step's tokens sit at positions lens + 1 and see lens + 2 keys
        rows = dev(torch.arange(n).int())
        split = dev(torch.zeros(n + 3).int())
        for kv_heads, sms in ((8, 148), (2, 148), (1, 132)):
            attention_bf16.decode_replan(split, context, rows, kv_heads, 3 * sms, 5, 32, own_length=False)
            want = split_length(n, longest + 2, kv_heads, sms)
            assert split[:n].cpu().tolist() == [want] * n, (n, longest, kv_heads)
            assert split[n:].eq(0).all()
        attention_bf16.decode_replan(split, context, rows, 8, 444, 5, 32, own_length=True)
        assert split[:n].cpu().tolist() == [split_length(1, int(x) + 2, own=True) for x in lens]
        # a full ring: the tokens are still handed over, no row is written
        counter.fill_(4)
        sampling.burst_advance(tokens, positions, context, dev(nxt), ring, counter)
        assert int(counter) == 5 and ring[[0, 1, 3]].eq(-7).all()


@pytest.mark.parametrize("n", [1000, 8191, 8192, 151936, 300001])
def test_argmax_first_maximum(n):
    """Short rows by one block, long rows shared among blocks: the first maximum either way,
    also where the maxima sit in different shares, and index 0 for a row without a number."""
    logits = torch.randn(7, n + 3, generator=torch.Generator().manual_seed(1))[:, :n].to(DEV)     # a pitch beside n
    logits[1, 7] = logits[1, n - 100] = 50.0
    logits[2, :] = 0.25
    logits[5, :] = float("nan")
    logits[6, :] = float("-inf")
    logits[6, : n // 2] = float("nan")
    out = ops().argmax_rows(logits).cpu().tolist()
    assert out == [int(logits[0].argmax()), 7, 0, int(logits[3].argmax()), int(logits[4].argmax()), 0, n // 2]


@pytest.mark.parametrize("vocab", [1000, 151936])
def test_sample_rows_draws_the_plain_sampler_tokens(vocab):
    from kipp_b200.kernels import sampling as ks
    g = torch.Generator().manual_seed(vocab)
    cases = [dict(temperature=0.0), dict(temperature=0.8), dict(temperature=1.3, top_k=5),
             dict(temperature=0.7, top_p=0.6), dict(temperature=1.0, min_p=0.2),
             dict(temperature=0.9, top_k=40, top_p=0.9, min_p=0.02), dict(temperature=0.25),
             dict(temperature=5.0, top_p=0.95), dict(temperature=1.0, top_k=1), dict(temperature=2.0, top_k=vocab + 5)]
    rows = len(cases)
    logits = (torch.randn(rows, vocab, generator=g) * 2.5)
    logits[:, 17] = logits[:, 200] = logits.max(dim=1).values - 0.25       # ties inside the candidates
    dev = logits.to(DEV)
    state = 99
    for trial in range(12):
        uni, want = [], []
        for r, c in enumerate(cases):
            tok, new_state = P.plain_sample(logits[r].numpy(), rng_state=state + r, **{"temperature": 0.0, **c})
            _, u = P.uniform_unit(state + r)
            uni.append(u)
            want.append(tok)
        f = lambda key, default, dt: torch.tensor([c.get(key, default) for c in cases], dtype=dt, device=DEV)
        got = ks.sample_rows(dev, f("temperature", 0.0, torch.float32), f("top_k", 0, torch.int32),
                             f("top_p", 1.0, torch.float32), f("min_p", 0.0, torch.float32),
                             torch.tensor(uni, dtype=torch.float64, device=DEV)).cpu().tolist()
        assert got == want, (trial, got, want)
        state = state * 7 + 13


def test_penalties_and_bias_match_the_reference_sampler():
    import json
    import os
    with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "operators.json")) as f:
        gold = json.load(f)["penalties"]
    from kipp_b200.kernels import sampling as ks
    logits = torch.tensor([gold["logits"], gold["logits"]], dtype=torch.float32, device=DEV)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)          # noqa: E731
    f32 = lambda v: torch.tensor(v, dtype=torch.float32, device=DEV)        # noqa: E731
    recent = gold["recent"]
    bias = {int(k): v for k, v in gold["bias"].items()}
    # row 0 has the penalties and the bias, row 1 none
    ks.apply_penalties(logits, i32([recent, [-1] * len(recent)]), i32([len(recent), 0]),
                       f32([gold["repetition"], 1.0]), f32([gold["presence"], 0.0]), f32([gold["frequency"], 0.0]),
                       i32([list(bias), [0] * len(bias)]), f32([list(bias.values()), [0.0] * len(bias)]),
                       i32([len(bias), 0]))
    out = ks.argmax_rows(logits).cpu().tolist()
    assert out[0] == gold["token"]                       # what kipp_sample_ex chose with the same settings
    assert out[1] == int(np.argmax(np.asarray(gold["logits"], dtype=np.float32))) and out[0] != out[1]


@pytest.mark.parametrize("case", [dict(D=128, nq=8, nkv=2, page=16, rot=True, norm=True, w16=True, window=None),
                                  dict(D=64, nq=6, nkv=3, page=8, rot=True, norm=True, w16=False, window=90),
                                  dict(D=128, nq=5, nkv=1, page=32, rot=False, norm=True, w16=True, window=None),
                                  dict(D=64, nq=16, nkv=1, page=16, rot=True, norm=False, w16=False, window=None)])
def test_decode_attention_fused_with_norm_rotation_and_cache_write(case):
    """A step of decoded tokens: the attention kernel that normalises, rotates and
    writes the new key and value itself against the two separate launches, on
    the same raw projection output; outputs and caches must agree (the norm's
    sum runs in another order: rounding only), and a run that does not write
    its cache leaves the pages alone."""
    from kipp_b200.kernels import attention_bf16
    D, nq, nkv, page, window = case["D"], case["nq"], case["nkv"], case["page"], case["window"]
    layout = [(700, 1), (15, 1), (16, 1), (255, 1), (1023, 1), (0, 1), (129, 1)]
    meta, table, _, kp, vp = attention_case(77, D, nq, nkv, page, layout, torch.bfloat16)
    T = meta.tokens
    g = torch.Generator().manual_seed(5)
    qkv = torch.randn(T, (nq + 2 * nkv) * D, generator=g).to(torch.bfloat16).to(DEV)
    wdt = torch.bfloat16 if case["w16"] else torch.float32
    qw = (1 + 0.2 * torch.randn(D, generator=g)).to(wdt).to(DEV) if case["norm"] else None
    kw = (1 + 0.2 * torch.randn(D, generator=g)).to(wdt).to(DEV) if case["norm"] else None
    rot = D if case["rot"] else 0
    inv = cos_sin = None
    if rot:
        i = torch.arange(D // 2, dtype=torch.float32)
        inv = torch.pow(torch.tensor(1e4, dtype=torch.float64), (-(2.0 * i) / D).double()).float().to(DEV)
        cos_sin = ops().rope_table(meta.positions, inv, T)
    assert attention_bf16.decode_fused_ok(meta, torch.bfloat16, nq, nkv, D, rot)
    st = status()
    # separate launches
    k1, v1 = kp.clone(), vp.clone()
    q = torch.zeros(T, nq, D, dtype=torch.bfloat16, device=DEV)
    ops().qk_norm_rope_write(qkv, q, k1, v1, qw, kw, 1e-6, inv, rot, meta.positions, meta.entry_of_token,
                             meta.block_tables[0], page, T, nq, nkv, D, True, st, cos_sin=cos_sin)
    want = torch.zeros_like(q)
    ops().attention(want, q, k1, v1, meta, meta.block_tables[0], page, nq, nkv, D, 1 / math.sqrt(D), window, st,
                    impl="mma")
    # one launch
    k2, v2 = kp.clone(), vp.clone()
    got = torch.full_like(q, 7.0)
    attention_bf16.decode_scratch(torch.device(DEV), T, nq, D).fill_(float("nan"))
    ops().attention_decode_fused(got, qkv, k2, v2, qw, kw, 1e-6, cos_sin, True, meta, meta.block_tables[0], page,
                                 nq, nkv, D, 1 / math.sqrt(D), window, st)
    assert st.tolist() == [0, 0, 0, 0]
    assert torch.equal(v1, v2)
    assert torch.allclose(k1.float(), k2.float(), rtol=1e-2, atol=1e-2)
    assert float((k1.float() - kp.float()).abs().sum()) > 0          # keys were written
    assert torch.allclose(got.float(), want.float(), rtol=2e-2, atol=2e-2)
    k4, v4 = kp.clone(), vp.clone()
    got4 = torch.full_like(q, 7.0)
    attention_bf16.decode_fused(got4, qkv, k4, v4, qw, kw, 1e-6, cos_sin, True, meta, meta.block_tables[0], page,
                                nq, nkv, D, 1 / math.sqrt(D), window, st, stream=False)
    assert torch.equal(k4, k2) and torch.equal(v4, v2)            # splits of a given length: the same cache
    assert torch.allclose(got4.float(), want.float(), rtol=2e-2, atol=2e-2)
    # reading another run's cache: nothing is written
    k3, v3 = k1.clone(), v1.clone()
    got3 = torch.zeros_like(q)
    ops().attention_decode_fused(got3, qkv, k3, v3, qw, kw, 1e-6, cos_sin, False, meta, meta.block_tables[0],
                                 page, nq, nkv, D, 1 / math.sqrt(D), window, st)
    assert torch.equal(k3, k1) and torch.equal(v3, v1)
    assert torch.allclose(got3.float(), want.float(), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("window", [None, 500])
@pytest.mark.parametrize("shape", [dict(D=128, nq=8, nkv=2, page=16), dict(D=64, nq=6, nkv=3, page=32),
                                   dict(D=128, nq=16, nkv=1, page=16)])
def test_decode_attention_dealt_out_as_a_stream(shape, window):
    """Many decoded tokens of very different lengths: the key tiles of all (token, kv head)
    pairs are dealt out in equal runs to one wave of CTAs, so runs end inside pairs and span
    several short ones; every token against the plain reference, and against the kernel
    that cuts each token into splits of its own.  A far key that stands out must be found
    wherever the cuts fall."""
    from kipp_b200.kernels import attention_bf16
    D, nq, nkv, page = shape["D"], shape["nq"], shape["nkv"], shape["page"]
    rng = random.Random(D + nq)
    layout = [(rng.choice([0, 1, 63, 64, 65, 200, 1000, 2500, 4000]) + rng.randrange(3), 1) for _ in range(70)]
    layout[5] = (6000, 1)
    meta, table, q, kp, vp = attention_case(31, D, nq, nkv, page, layout, torch.bfloat16)
    # one key far back in the longest request that the query of that token points at
    e, far = 5, 777
    pg, slot = int(table[e, far // page]), far % page
    kp[pg, :, slot, :] = 0
    kp[pg, :, slot, 0] = 30.0
    q[e, :, :] = 0
    q[e, :, 0] = 30.0
    st = status()
    attention_bf16.decode_scratch(torch.device(DEV), meta.tokens, nq, D).fill_(float("nan"))
    out = torch.full_like(q, 9.0)
    attention_bf16.run("mma", out, q, kp, vp, meta, meta.block_tables[0], page, nq, nkv, D, 1 / math.sqrt(D), window, st)
    ref = attention_ref(meta, table, q, kp, vp, layout, page, window, 1 / math.sqrt(D))
    assert torch.allclose(out.double().cpu(), ref, rtol=2e-2, atol=2e-2)
    if window is None:                           # the far key takes all the weight
        assert torch.allclose(out[e].float().cpu(), vp[pg, :, slot, :].float().cpu().repeat_interleave(nq // nkv, 0),
                              rtol=2e-2, atol=2e-2)
    out1 = torch.full_like(q, 9.0)
    attention_bf16.run("mma", out1, q, kp, vp, meta, meta.block_tables[0], page, nq, nkv, D, 1 / math.sqrt(D), window,
                       st, stream=False)
    assert torch.allclose(out1.float(), out.float(), rtol=2e-2, atol=2e-2)
    assert st.tolist() == [0, 0, 0, 0]


def test_a_bounded_wait_runs_out_and_reports():
    """The give-up branch of the mbarrier wait every tensor-core kernel uses
    (csrc/mbarrier.cuh), run by a probe kernel on a barrier nothing arrives at, with
    a limit of some ten microseconds: the kernel returns by itself, the status word
    the engine reads is set, and the wait lasted as long as its limit."""
    import ctypes
    from kipp_b200.csrc.build import load_library
    lib = load_library("wait_probe")
    lib.kipp_wait_probe.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p]
    lib.kipp_wait_probe.restype = ctypes.c_int
    st = status()
    waited = torch.zeros(1, dtype=torch.int64, device=DEV)
    limit = 20_000
    rc = lib.kipp_wait_probe(st.data_ptr(), waited.data_ptr(), limit, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert rc == 0
    assert st.tolist() == [0, 1, 0, 0]
    assert limit <= int(waited) < 200 * limit
