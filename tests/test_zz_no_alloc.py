"""tie_attention_split_noalloc, the entry point for callers that cannot allocate device memory,
called through its exported C symbol and compared with tie_attention_split (which takes the
caller's scratch buffer) on the same inputs.

It is for embedders that run inside a fixed memory budget or are handed their buffers by a host
application: they have no scratch buffer to give. The test makes two calls in a row with
different shapes, so the second call finds the first one's leftovers in the built-in array, and
checks the refusal of a problem that does not fit it. The file sorts last on purpose: a run
that stops at the first failure has then run every other test already. It passes alone in a
fresh process (its first call does the per-device set-up) and after the other tests.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(seed, n_seqs, Hq, Hkv, Dh, page, ctx_max, dtype):
    rng = np.random.default_rng(seed)
    ctx = rng.integers(1, ctx_max, n_seqs)
    pages_per = -(-int(ctx.max()) // page)
    n_pages = n_seqs * pages_per + 3
    g = torch.Generator(device="cuda").manual_seed(seed)
    kc = torch.randn(n_pages, Hkv, page, Dh, device="cuda", generator=g).to(dtype)
    vc = torch.randn(n_pages, Hkv, page, Dh, device="cuda", generator=g).to(dtype)
    q = torch.randn(n_seqs, Hq * Dh, device="cuda", generator=g).to(dtype)
    tables = torch.from_numpy(rng.permutation(n_pages)[:n_seqs * pages_per].reshape(n_seqs, pages_per).astype(np.int32)).cuda()
    query_start = torch.arange(n_seqs + 1, dtype=torch.int32, device="cuda")
    context_lens = torch.from_numpy(ctx.astype(np.int32)).cuda()
    seq_list = torch.arange(n_seqs, dtype=torch.int32, device="cuda")
    return q, kc, vc, tables, query_start, context_lens, seq_list


def _noalloc(lib, q, kc, vc, out, tables, query_start, context_lens, seq_list, Hq, Hkv, Dh, scale, split_keys, max_splits,
             window=0):
    from tiny_inference_engine_b200.ops import dtype_code
    P, I, L, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
    fn = lib.tie_attention_split_noalloc
    fn.argtypes = [I, P, L, P, P, P, P, P, P, I, I, I, I, I, I, I, F, P, I, I, I, P]
    fn.restype = I
    return fn(dtype_code(q), q.data_ptr(), q.stride(0), kc.data_ptr(), vc.data_ptr(), out.data_ptr(), query_start.data_ptr(),
              context_lens.data_ptr(), tables.data_ptr(), tables.shape[1], context_lens.numel(), Hq, Hkv, Dh, kc.shape[2],
              window, scale, seq_list.data_ptr(), seq_list.numel(), split_keys, max_splits, torch.cuda.current_stream().cuda_stream)


def test_no_alloc_entry_point_matches_the_one_with_caller_scratch():
    from tiny_inference_engine_b200 import ops
    from tiny_inference_engine_b200.ops.library import library
    lib = library()
    for seed, (n_seqs, Hq, Hkv, Dh, page, ctx_max, dtype, split_keys) in enumerate([
            (5, 8, 2, 64, 16, 700, torch.bfloat16, 128),      # first call: does the set-up on this device
            (3, 6, 3, 48, 8, 300, torch.float32, 64)]):       # second call: other shapes, stale partials in the array
        q, kc, vc, tables, query_start, context_lens, seq_list = _case(seed, n_seqs, Hq, Hkv, Dh, page, ctx_max, dtype)
        max_splits = -(-ctx_max // split_keys)
        scale = 1.0 / np.sqrt(Dh)
        want = torch.zeros(n_seqs, Hq * Dh, device="cuda", dtype=dtype)
        scratch = torch.empty(ops.attention_split_scratch_floats(n_seqs, Hq, Dh, max_splits), device="cuda")
        ops.attention_split(q, kc, vc, want, query_start, context_lens, tables, Hq, Hkv, Dh, scale, seq_list, n_seqs,
                            split_keys, max_splits, scratch)
        got = torch.full_like(want, float("nan"))
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]     # cudaMemGetInfo: it sees every allocation on the device, not torch's alone
        status = _noalloc(lib, q, kc, vc, got, tables, query_start, context_lens, seq_list, Hq, Hkv, Dh, scale, split_keys,
                          max_splits)
        torch.cuda.synchronize()
        assert status == 0, lib.tie_last_error().decode()
        if seed > 0:                                   # the first call on a device may load the kernels' code
            assert torch.cuda.mem_get_info()[0] >= free_before, "the call took device memory"
        assert torch.equal(got, want), f"call {seed}: the same kernels on the same data give the same bits"


def test_no_alloc_entry_point_against_the_plain_attention_with_a_window_a_subset_and_an_empty_sequence():
    """Not against the entry point with caller scratch (the two share kernels and could share a fault) but against the
    plain float64 attention: a window, a seq_list that leaves sequences out, one sequence without keys, more splits
    allowed than any sequence needs, and an output filled with NaN so that a row never written shows."""
    import plain_qwen3 as plain
    from tiny_inference_engine_b200.ops.library import library
    lib = library()
    rng = np.random.default_rng(5)
    Hq, Hkv, Dh, page, window, split_keys, max_splits = 6, 2, 32, 8, 150, 64, 9
    ctx = [400, 0, 77, 151, 9]
    chosen = [0, 1, 3, 4]                                # sequence 2 is left out
    n_pages = sum(-(-c // page) for c in ctx) + 4
    order = rng.permutation(n_pages)
    kc, vc = np.zeros((n_pages, Hkv, page, Dh), dtype=np.float32), np.zeros((n_pages, Hkv, page, Dh), dtype=np.float32)
    tables = np.zeros((len(ctx), max(-(-c // page) for c in ctx) + 2), dtype=np.int32)
    ks, vs, used = [], [], 0
    for i, n in enumerate(ctx):
        k, v = rng.standard_normal((n, Hkv, Dh)).astype(np.float32), rng.standard_normal((n, Hkv, Dh)).astype(np.float32)
        for j in range(n):
            if j % page == 0:
                tables[i, j // page] = order[used]
                used += 1
            kc[tables[i, j // page], :, j % page], vc[tables[i, j // page], :, j % page] = k[j], v[j]
        ks.append(k), vs.append(v)
    q = rng.standard_normal((len(ctx), Hq * Dh)).astype(np.float32)
    out = torch.full((len(ctx), Hq * Dh), float("nan"), device="cuda")
    cuda = lambda a, dt=torch.float32: torch.from_numpy(np.ascontiguousarray(a)).to("cuda").to(dt)
    status = _noalloc(lib, cuda(q), cuda(kc), cuda(vc), out, cuda(tables, torch.int32), cuda(np.arange(len(ctx) + 1), torch.int32),
                      cuda(np.array(ctx), torch.int32), cuda(np.array(chosen), torch.int32), Hq, Hkv, Dh,
                      float(1 / np.sqrt(np.float32(Dh))), split_keys, max_splits, window=window)
    torch.cuda.synchronize()
    assert status == 0, lib.tie_last_error().decode()
    got = out.cpu().numpy()
    assert np.isnan(got[2]).all()                        # not in the list: not touched
    assert (got[1] == 0).all()                           # no keys: zeros
    for i in (0, 3, 4):
        n = ctx[i]
        qfull = np.zeros((n, Hq * Dh))
        qfull[-1] = q[i]
        want = plain.causal_attention(qfull, ks[i].reshape(n, -1), vs[i].reshape(n, -1), Hq, Hkv, Dh, window)[-1]
        assert np.abs(got[i] - want).max() <= 2e-5 * np.abs(want).max(), f"sequence {i}"


def test_no_alloc_entry_point_refuses_what_does_not_fit():
    from tiny_inference_engine_b200.ops.library import library
    lib = library()
    q, kc, vc, tables, query_start, context_lens, seq_list = _case(9, 64, 32, 8, 128, 16, 100, torch.bfloat16)
    out = torch.zeros(64, 32 * 128, device="cuda", dtype=torch.bfloat16)
    status = _noalloc(lib, q, kc, vc, out, tables, query_start, context_lens, seq_list, 32, 8, 128, 0.1, 64, 64)
    assert status == 1 and "exceed the built-in" in lib.tie_last_error().decode()
    torch.cuda.synchronize()
    assert not out.any()
