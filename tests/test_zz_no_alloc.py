"""The decode-attention entry point that allocates nothing
(kipp_attn_decode_mma_noalloc, csrc/attention_decode_noalloc.h).

Some callers cannot give the kernel a scratch buffer because they may not
allocate device memory where they run (a hook inside another framework, a
process whose memory is fixed and given out at start-up).  For them the scratch
is a fixed array inside the library.  This test calls that entry point through
its exported C symbol, twice in a row on different inputs, and checks each
result against the ordinary entry point, which takes its scratch from the
caller, and against a plain float64 attention.  The file sorts last so that a run that stops at the first failure has
run everything else before.
"""
import ctypes
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
MAX_SPLITS = 32


def make_case(seed, n_q, n_kv, D, page, contexts):
    """Single decoded tokens with ``contexts`` cached tokens each, pages taken
    from a shuffled pool."""
    from gpu_util import pack_meta as pack_step
    from kipp_b200.engine.batch import StepEntry
    g = torch.Generator().manual_seed(seed)
    entries = [StepEntry(i, [0], []) for i in range(len(contexts))]
    need = [-(-(c + 1) // page) for c in contexts]
    width = max(need)
    n_pages = sum(need) + 2
    perm = torch.randperm(n_pages, generator=g).tolist()
    table = np.full((len(contexts), width), -1, dtype=np.int32)
    at = 0
    for i, k in enumerate(need):
        table[i, :k] = perm[at:at + k]
        at += k
    meta = pack_step(entries, list(contexts), list(range(len(contexts))), [table], torch.device(DEV))
    q = torch.randn(len(contexts), n_q, D, generator=g).to(torch.bfloat16).to(DEV)
    kp = torch.randn(n_pages, n_kv, page, D, generator=g).to(torch.bfloat16).to(DEV)
    vp = torch.randn(n_pages, n_kv, page, D, generator=g).to(torch.bfloat16).to(DEV)
    return meta, q, kp, vp, table


def plain_attention_of(meta, table, q, kp, vp, contexts, page, window, D):
    """Softmax attention of every decoded token over its own keys, in float64."""
    from test_gpu_kernels import attention_ref
    return attention_ref(meta, table, q, kp, vp, [(c, 1) for c in contexts], page, window, 1 / math.sqrt(D))


def reference_entry(meta, q, kp, vp, n_q, n_kv, D, page, window):
    """The existing entry point: scratch comes from the caller (torch); every token cut into
    splits of the given length, as the entry point without allocation cuts them."""
    from kipp_b200.kernels import attention_bf16
    out = torch.zeros_like(q)
    attention_bf16.run("mma", out, q, kp, vp, meta, meta.block_tables[0], page, n_q, n_kv, D, 1 / math.sqrt(D),
                       window, torch.zeros(4, dtype=torch.int32, device=DEV), stream=False)
    return out


def noalloc_symbol():
    from kipp_b200.csrc.build import compile_library
    lib = ctypes.CDLL(compile_library("attention_decode_noalloc"))
    fn = lib.kipp_attn_decode_mma_noalloc            # the exported C symbol
    vp, ci = ctypes.c_void_p, ctypes.c_int
    fn.argtypes = [vp, vp, vp, vp, vp, vp, vp, ci, ci, vp, ci, ci, ci, ci, ctypes.c_float, ci, ci, vp, vp]
    fn.restype = ci
    need = lib.kipp_attn_decode_noalloc_scratch_bytes
    need.argtypes = [ci, ci, ci, ci]
    need.restype = ctypes.c_longlong
    return fn, need


def call_noalloc(fn, meta, q, kp, vp, n_q, n_kv, D, page, window):
    out = torch.zeros_like(q)
    bt = meta.block_tables[0]
    rc = fn(out.data_ptr(), q.data_ptr(), kp.data_ptr(), vp.data_ptr(), meta.q_start.data_ptr(),
            meta.context_len.data_ptr(), bt.data_ptr(), bt.shape[1], page, meta.decode_rows.data_ptr(),
            meta.n_decode, n_q, n_kv, D, 1 / math.sqrt(D), int(window or 0), MAX_SPLITS,
            meta.decode_split_keys.data_ptr(), torch.cuda.current_stream().cuda_stream)
    return rc, out


def test_two_calls_in_a_row_match_the_entry_point_that_is_given_scratch():
    fn, need = noalloc_symbol()
    n_q, n_kv, D, page = 8, 2, 128, 16
    before = torch.cuda.memory_allocated(DEV)
    results = []
    for seed, contexts, window in ((1, [700, 15, 16, 255, 1023], None), (2, [40, 900, 333], 100)):
        meta, q, kp, vp, table = make_case(seed, n_q, n_kv, D, page, contexts)
        want = reference_entry(meta, q, kp, vp, n_q, n_kv, D, page, window)
        held = torch.cuda.memory_allocated(DEV)
        rc, got = call_noalloc(fn, meta, q, kp, vp, n_q, n_kv, D, page, window)
        torch.cuda.synchronize()
        assert rc == 0
        # the same kernels in the same order: equal within the tolerance of the kernel tests
        assert torch.allclose(got.float(), want.float(), rtol=2e-2, atol=2e-2)
        assert torch.equal(got, want)
        assert float(got.float().abs().sum()) > 0
        # and it is the attention of these queries over these pages, whatever the other entry point says
        plain = plain_attention_of(meta, table, q, kp, vp, contexts, page, window, D)
        assert torch.allclose(got.double().cpu(), plain, rtol=2e-2, atol=2e-2)
        # torch allocated only this test's own output tensor around the call
        assert torch.cuda.memory_allocated(DEV) - held <= got.numel() * 2 + 512
        results.append(got)
    assert results[0].shape != results[1].shape          # the second call did not reuse the first's sizes
    # sizes beyond the built-in scratch are refused before anything runs
    assert need(8, n_q, D, MAX_SPLITS) == 8 * n_q * MAX_SPLITS * (D + 2) * 4
    assert need(4096, 64, 128, MAX_SPLITS) > (16 << 20)
    meta, q, kp, vp, _ = make_case(3, 64, 2, 128, page, [10] * 40)
    rc, out = call_noalloc(fn, meta, q, kp, vp, 64, 2, 128, page, None)
    assert rc == -4 and float(out.float().abs().sum()) == 0.0
