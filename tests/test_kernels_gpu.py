"""Each CUDA kernel alone against the plain implementation's function for the same op, at sizes the
tiny models do not use: widths and vocabularies that are no power of two, head sizes in steps
of 16, odd numbers of heads and groups, scattered pages."""
import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from conftest import rel_err

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 2e-5, "bfloat16": 1.2e-2}   # one kernel: a few float32 roundings, or one bfloat16 rounding of the output


def dev(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a)).to("cuda").to(dtype)


def host(t):
    return t.float().cpu().numpy()


def as_stored(a, dtype):
    """What the kernel sees: the values after rounding to the storage dtype."""
    return plain.round_bf16(a.astype(np.float32)) if dtype == "bfloat16" else a.astype(np.float32)


@pytest.fixture(scope="module")
def ops():
    from tiny_inference_engine_b200 import ops
    return ops


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embed(ops, dtype):
    """Widths that let a thread move 16 bytes of the table at a time, and one that does not."""
    rng = np.random.default_rng(0)
    for width in (72, 75, 4096):
        table = as_stored(rng.standard_normal((311, width)), dtype)
        ids = rng.integers(0, 311, 37)
        out = torch.full((37, width), float("nan"), device="cuda")
        ops.embed(dev(table, DT[dtype]), dev(ids, torch.int32), out)
        assert np.array_equal(host(out), plain.embed(table, ids).astype(np.float32))


def test_scatter_ids(ops):
    """tokens[dst[i]] = ids[src[i]] for the first n pairs; everything else is left as it is."""
    rng = np.random.default_rng(5)
    tokens = rng.integers(0, 1000, 700).astype(np.int32)
    ids = rng.integers(0, 1000, 300).astype(np.int32)
    dst = rng.permutation(700)[:300].astype(np.int32)
    src = rng.integers(0, 300, 300).astype(np.int32)
    for n in (0, 1, 129, 300):
        t = dev(tokens, torch.int32)
        ops.scatter_ids(t, dev(dst, torch.int32), dev(src, torch.int32), dev(ids, torch.int32), n)
        want = tokens.copy()
        want[dst[:n]] = ids[src[:n]]
        assert np.array_equal(host(t), want)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("dim", [72, 1000, 5120])
def test_add_rmsnorm(ops, dtype, dim):
    rng = np.random.default_rng(dim)
    x = rng.standard_normal((9, dim)).astype(np.float32) * 3
    delta = as_stored(rng.standard_normal((9, dim)), dtype)
    w = (1 + 0.1 * rng.standard_normal(dim)).astype(np.float32)
    xd, out = dev(x), torch.empty(9, dim, device="cuda", dtype=DT[dtype])
    ops.add_rmsnorm(xd, dev(delta, DT[dtype]), dev(w), 1e-5, out)
    want_x = x.astype(np.float64) + delta
    assert np.abs(host(xd) - want_x).max() < 1e-6 * np.abs(want_x).max()        # the residual sum is float32
    assert rel_err(host(out), plain.rms_norm(want_x, w, 1e-5)) < TOL[dtype]
    # without a delta x is untouched; with rows only those rows come out and x is not written
    x2 = dev(x)
    ops.add_rmsnorm(x2, None, dev(w), 1e-5, out)
    assert np.array_equal(host(x2), x) and rel_err(host(out), plain.rms_norm(x, w, 1e-5)) < TOL[dtype]
    rows = np.array([7, 0, 7, 3])
    out4 = torch.empty(4, dim, device="cuda", dtype=DT[dtype])
    x3 = dev(x)
    ops.add_rmsnorm(x3, dev(delta, DT[dtype]), dev(w), 1e-5, out4, rows=dev(rows, torch.int32))
    assert np.array_equal(host(x3), x) and rel_err(host(out4), plain.rms_norm(want_x[rows], w, 1e-5)) < TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rmsnorm_rows_on_a_strided_view(ops, dtype):
    rng = np.random.default_rng(1)
    x = as_stored(rng.standard_normal((20, 200)), dtype)
    w = (1 + 0.1 * rng.standard_normal(48)).astype(np.float32)
    xd = dev(x, DT[dtype])
    view = xd[:, 16:64]
    ops.rmsnorm_rows(view, dev(w), 3e-6, view)
    got = host(xd)
    assert rel_err(got[:, 16:64], plain.rms_norm(x[:, 16:64], w, 3e-6)) < TOL[dtype]
    assert np.array_equal(got[:, :16], x[:, :16]) and np.array_equal(got[:, 64:], x[:, 64:])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_silu_mul(ops, dtype):
    rng = np.random.default_rng(2)
    gu = as_stored(rng.standard_normal((11, 2 * 203)) * 4, dtype)
    out = torch.empty(11, 203, device="cuda", dtype=DT[dtype])
    ops.silu_mul(dev(gu, DT[dtype]), out)
    assert rel_err(host(out), plain.swiglu(gu[:, :203], gu[:, 203:])) < TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,head_dim,theta", [(3, 48, 1e4), (5, 16, 1e6), (2, 128, 5e5)])
def test_rope(ops, dtype, heads, head_dim, theta):
    rng = np.random.default_rng(3)
    x = as_stored(rng.standard_normal((13, heads * head_dim)), dtype)
    pos = np.array([0, 1, 2, 3, 17, 100, 1000, 4095, 40000, 5, 6, 7, 8])
    xd = dev(x, DT[dtype])
    ops.rope(xd, dev(pos, torch.int32), dev(plain.rope_inv_freq(theta, head_dim)), heads, head_dim)
    assert rel_err(host(xd), plain.rope_neox(x, pos, heads, head_dim, theta)) < TOL[dtype]
    assert np.array_equal(host(xd)[0], x[0])     # position 0 is the identity


def paged_cache(rng, dtype, n_tokens_per_seq, kv_heads, head_dim, page, n_pages):
    """Keys and values of several sequences scattered over shuffled pages."""
    pages = rng.permutation(n_pages)
    kc = np.zeros((n_pages, kv_heads, page, head_dim), dtype=np.float32)
    vc = np.zeros_like(kc)
    tables, ks, vs, used = [], [], [], 0
    for n in n_tokens_per_seq:
        nb = -(-n // page)
        tab = pages[used:used + nb]
        used += nb
        k = as_stored(rng.standard_normal((n, kv_heads, head_dim)), dtype)
        v = as_stored(rng.standard_normal((n, kv_heads, head_dim)), dtype)
        for j in range(n):
            kc[tab[j // page], :, j % page] = k[j]
            vc[tab[j // page], :, j % page] = v[j]
        tables.append(tab), ks.append(k), vs.append(v)
    mb = max(len(t) for t in tables) + 3
    bt = np.zeros((len(tables), mb), dtype=np.int32)
    for i, t in enumerate(tables):
        bt[i, :len(t)] = t
    return kc, vc, bt, ks, vs


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T", [21, 300])
@pytest.mark.parametrize("Hq,Hkv,Dh", [(6, 3, 48), (4, 2, 64), (5, 3, 64), (8, 2, 128), (3, 1, 128), (2, 1, 256)])
def test_kv_append_and_fused_norm_rope_append(ops, dtype, T, Hq, Hkv, Dh):
    """Head size 48 runs the general kernel, 64 / 128 / 256 the one that holds a head in a warp's registers, and
    with hundreds of tokens the one that works on a token's heads side by side (odd head counts put a query head
    and a key head, or a value head and nothing, into one warp)."""
    rng = np.random.default_rng(4)
    page = 8
    n_pages = max(12, T // page + 5)
    qkv = as_stored(rng.standard_normal((T, (Hq + 2 * Hkv) * Dh)), dtype)
    qw, kw = (1 + 0.2 * rng.standard_normal(Dh)).astype(np.float32), (1 + 0.2 * rng.standard_normal(Dh)).astype(np.float32)
    pos = rng.integers(0, 3000, T)
    slots = rng.permutation(n_pages * page)[:T]
    slots[5] = -1                                  # a padding row writes nothing
    kc = torch.zeros(n_pages, Hkv, page, Dh, device="cuda", dtype=DT[dtype])
    vc = torch.zeros_like(kc)
    inv = plain.rope_inv_freq(1e6, Dh)
    qd = dev(qkv, DT[dtype])
    ops.qk_norm_rope_append(qd, dev(qw), dev(kw), 1e-6, 1e-5, dev(inv), dev(pos, torch.int32), dev(slots, torch.int32),
                            kc, vc, Hq, Hkv, Dh)
    q, k, v = qkv[:, :Hq * Dh], qkv[:, Hq * Dh:(Hq + Hkv) * Dh], qkv[:, (Hq + Hkv) * Dh:]
    want_q = plain.rope_neox(plain.rms_norm(q.reshape(T * Hq, Dh), qw, 1e-6).reshape(T, -1), pos, Hq, Dh, 1e6)
    want_k = plain.rope_neox(plain.rms_norm(k.reshape(T * Hkv, Dh), kw, 1e-5).reshape(T, -1), pos, Hkv, Dh, 1e6)
    assert rel_err(host(qd)[:, :Hq * Dh], want_q) < TOL[dtype]
    got_k, got_v = host(kc), host(vc)
    for t in range(T):
        if slots[t] < 0:
            continue
        p, o = slots[t] // page, slots[t] % page
        assert rel_err(got_k[p, :, o].reshape(1, -1), want_k[t].reshape(1, -1)) < TOL[dtype]
        assert np.array_equal(got_v[p, :, o].reshape(-1), v[t])
    written = {(s // page, s % page) for s in slots if s >= 0}
    for p in range(n_pages):
        for o in range(page):
            if (p, o) not in written:
                assert not got_k[p, :, o].any() and not got_v[p, :, o].any()
    # the unfused kernel writes the same places
    kc2, vc2 = torch.zeros_like(kc), torch.zeros_like(vc)
    ops.kv_append(dev(want_k, DT[dtype]), dev(v, DT[dtype]), dev(slots, torch.int32), kc2, vc2)
    assert np.array_equal(host(vc2), got_v)
    # without norm weights and without rotation the fused kernel only copies
    q2 = dev(qkv, DT[dtype])
    ops.qk_norm_rope_append(q2, None, None, 0, 0, None, dev(pos, torch.int32), dev(slots, torch.int32), kc2, vc2, Hq, Hkv, Dh)
    assert np.array_equal(host(q2), qkv)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("M,N,K", [(1, 503, 96), (3, 72, 200), (8, 1000, 520), (13, 311, 144), (70, 130, 75), (200, 96, 1000)])
def test_gemm_simt(ops, dtype, M, N, K):
    rng = np.random.default_rng(M * N)
    a, w = as_stored(rng.standard_normal((M, K)), dtype), as_stored(rng.standard_normal((N, K)), dtype)
    out = torch.empty(M, N, device="cuda", dtype=DT[dtype])
    ops.gemm_simt(dev(a, DT[dtype]), dev(w, DT[dtype]), out)
    assert rel_err(host(out), plain.linear(a, w)) < TOL[dtype]
    if dtype == "bfloat16":                         # logits come out in float32
        out32 = torch.empty(M, N, device="cuda")
        ops.gemm_simt(dev(a, DT[dtype]), dev(w, DT[dtype]), out32)
        assert rel_err(host(out32), plain.linear(a, w)) < 2e-5


def dense_reference(q, k, v, Hq, Hkv, Dh, n_new, window=0):
    """The last n_new rows of causal attention over all of k, v."""
    n = k.shape[0]
    qfull = np.zeros((n, Hq * Dh))
    qfull[n - n_new:] = q
    return plain.causal_attention(qfull, k.reshape(n, -1), v.reshape(n, -1), Hq, Hkv, Dh, window)[n - n_new:]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("Hq,Hkv,Dh,page,window", [(4, 2, 16, 16, 0), (8, 1, 32, 8, 0), (3, 3, 48, 32, 0), (6, 2, 128, 16, 0),
                                                  (5, 5, 80, 4, 0), (4, 1, 64, 16, 37)])
def test_paged_attention_rows_and_split(ops, dtype, Hq, Hkv, Dh, page, window):
    """Mixed batch: two sequences bring portions over a cached prefix, three bring one token;
    pages are scattered. Rows kernel for the first, split kernel for the others."""
    rng = np.random.default_rng(Hq * Dh)
    ctx = [45, 300, 1, 33, 700]          # tokens in the cache after the step
    new = [45, 17, 1, 1, 1]              # of which this step brings
    kc, vc, bt, ks, vs = paged_cache(rng, dtype, ctx, Hkv, Dh, page, 120 * 16 // page)
    T = sum(new)
    q = as_stored(rng.standard_normal((T, Hq * Dh)), dtype)
    qs = np.concatenate([[0], np.cumsum(new)])
    scale = 1.0 / np.sqrt(Dh)
    want = np.concatenate([dense_reference(q[qs[i]:qs[i + 1]], ks[i], vs[i], Hq, Hkv, Dh, new[i], window) for i in range(5)])
    seq_of_row = np.repeat(np.arange(5), new)
    out = torch.zeros(T, Hq * Dh, device="cuda", dtype=DT[dtype])
    args = (dev(kc, DT[dtype]), dev(vc, DT[dtype]), out)
    meta = (dev(qs, torch.int32), dev(np.array(ctx), torch.int32), dev(bt, torch.int32))
    ops.attention_rows(dev(q, DT[dtype]), *args, dev(seq_of_row, torch.int32), *meta, Hq, Hkv, Dh, scale, window)
    assert rel_err(host(out), want) < TOL[dtype]
    # the same single-token sequences through the split kernel, with splits of 64 keys
    out2 = torch.zeros_like(out)
    n_multi = new[0] + new[1]
    scratch = torch.empty(ops.attention_split_scratch_floats(3, Hq, Dh, 11), device="cuda")
    ops.attention_split(dev(q, DT[dtype]), *args[:2], out2, *meta, Hq, Hkv, Dh, scale, dev(np.array([2, 3, 4]), torch.int32),
                        3, 64, 11, scratch, window)
    assert rel_err(host(out2)[n_multi:], want[n_multi:]) < TOL[dtype]
    assert not host(out2)[:n_multi].any()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("far", [0, 15, 16, 31, 32, 255, 256, 257, 511, 512, 1022, 1023])
def test_one_far_key_among_a_thousand_is_found(ops, dtype, far):
    """The query matches exactly one key, at a page's edge, a chunk's edge, a split's edge, the
    first key, the last: the output must be that key's value row. Random data would hide a key
    that is skipped or read from the wrong page: it would move the result by a thousandth."""
    rng = np.random.default_rng(far)
    Hq, Hkv, Dh, page, n = 4, 2, 32, 16, 1024
    kc, vc, bt, ks, vs = paged_cache(rng, dtype, [n], Hkv, Dh, page, 80)
    q = np.zeros((1, Hq * Dh), dtype=np.float32)
    for h in range(Hq):
        q[0, h * Dh:(h + 1) * Dh] = 8.0 * ks[0][far, h // 2] * np.sqrt(Dh)   # score ~ 8 * |k|^2 ~ 256 above the rest
    q = as_stored(q, dtype)
    meta = (dev(np.array([0, 1]), torch.int32), dev(np.array([n]), torch.int32), dev(bt, torch.int32))
    one_hot = np.concatenate([vs[0][far, h // 2] for h in range(Hq)])[None]
    want = dense_reference(q, ks[0], vs[0], Hq, Hkv, Dh, 1)
    assert np.abs(want - one_hot).max() < 1e-3      # the far key really holds all the weight
    for split in (False, True):
        out = torch.zeros(1, Hq * Dh, device="cuda", dtype=DT[dtype])
        if split:
            scratch = torch.empty(ops.attention_split_scratch_floats(1, Hq, Dh, 4), device="cuda")
            ops.attention_split(dev(q, DT[dtype]), dev(kc, DT[dtype]), dev(vc, DT[dtype]), out, *meta, Hq, Hkv, Dh,
                                1 / np.sqrt(Dh), dev(np.array([0]), torch.int32), 1, 256, 4, scratch)
        else:
            ops.attention_rows(dev(q, DT[dtype]), dev(kc, DT[dtype]), dev(vc, DT[dtype]), out,
                               dev(np.array([0]), torch.int32), *meta, Hq, Hkv, Dh, 1 / np.sqrt(Dh))
        assert np.abs(host(out) - want).max() < 1e-2, f"split={split}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_window_edge(ops, dtype):
    """With a window of 40 the key at position pos-39 counts and the one at pos-40 does not."""
    rng = np.random.default_rng(9)
    Hq, Hkv, Dh, page, n, window = 2, 1, 32, 8, 200, 40
    kc, vc, bt, ks, vs = paged_cache(rng, dtype, [n], Hkv, Dh, page, 40)
    meta = (dev(np.array([0, 1]), torch.int32), dev(np.array([n]), torch.int32), dev(bt, torch.int32))
    for target, inside in ((n - 1 - 39, True), (n - 1 - 40, False)):
        q = as_stored(np.tile(8.0 * ks[0][target, 0] * np.sqrt(Dh), Hq)[None], dtype)
        out = torch.zeros(1, Hq * Dh, device="cuda", dtype=DT[dtype])
        ops.attention_rows(dev(q, DT[dtype]), dev(kc, DT[dtype]), dev(vc, DT[dtype]), out, dev(np.array([0]), torch.int32),
                           *meta, Hq, Hkv, Dh, 1 / np.sqrt(Dh), window)
        hit = np.abs(host(out)[0, :Dh] - vs[0][target, 0]).max() < 1e-2
        assert hit == inside


def test_sampling_kernel_greedy_and_temperature(ops):
    rng = np.random.default_rng(5)
    R, V = 7, 1531
    z = (rng.standard_normal((R, V)) * 2).astype(np.float32)
    z[2, 100] = z[2, 900] = z[2].max() + 1          # a tie goes to the lowest id
    z[3, 5] = np.inf
    out = torch.empty(R, dtype=torch.int32, device="cuda")
    ops.sample(dev(z), out)
    assert out.tolist() == [plain.sample(z[r]) for r in range(R)] and out[2].item() == 100
    temps = np.array([0.8, 0.0, 1.0, 0.7, 1e-45, 2.5, 0.3], dtype=np.float32)
    with np.errstate(divide="ignore", over="ignore"):
        inv = np.where(temps > 0, np.float32(1) / temps, 0).astype(np.float32)
    inv[~np.isfinite(inv)] = 0
    seeds = np.array([7, 1, 2 ** 63 + 11, 4, 5, 6, 2 ** 40], dtype=np.uint64)
    for counter in (0, 1, 2, 1000, 2 ** 33):
        ctr = np.full(R, counter, dtype=np.int64)
        ops.sample(dev(z), out, dev(inv), torch.from_numpy(seeds.view(np.int64)).cuda(), dev(ctr, torch.int64))
        want = [plain.sample(z[r], float(temps[r]), u=plain.uniform_for(int(seeds[r]), counter)) for r in range(R)]
        assert out.tolist() == want


def test_sampling_kernel_frequencies(ops):
    z = np.tile(np.array([[0.0, 1.0, 2.0, -30.0, 0.5]], dtype=np.float32), (2000, 1))
    out = torch.empty(2000, dtype=torch.int32, device="cuda")
    inv = np.full(2000, 1 / 0.8, dtype=np.float32)
    ops.sample(dev(z), out, dev(inv), dev(np.full(2000, 3), torch.int64), dev(np.arange(2000), torch.int64))
    p = np.exp(z[0] / 0.8 - (z[0] / 0.8).max())
    p /= p.sum()
    assert np.abs(np.bincount(out.cpu().numpy(), minlength=5) / 2000 - p).max() < 0.03


def _filtered_case(ops, z, rows, counter, one_cta=False):
    """rows: (temperature, top_k, top_p, seed) for each row of z; the kernels against the sampler on the host."""
    from tiny_inference_engine_b200.sampling import SamplingParams
    from host_sampler import sample_host
    R = len(rows)
    params = [SamplingParams(temperature=t, top_k=k, top_p=p, seed=s) for t, k, p, s in rows]
    inv = np.array([q.inv_temperature() for q in params], dtype=np.float32)
    seeds = np.array([q.seed for q in params], dtype=np.uint64)
    out = torch.full((R,), -1, dtype=torch.int32, device="cuda")
    ops.sample(dev(z), out, dev(inv), torch.from_numpy(seeds.view(np.int64)).cuda(), dev(np.full(R, counter), torch.int64),
               dev(np.array([q.top_k for q in params]), torch.int32), dev(np.array([q.top_p for q in params], dtype=np.float32)),
               one_cta=one_cta)
    want = [sample_host(z[r], params[r], counter) for r in range(R)]
    assert out.tolist() == want, [(rows[r], out[r].item(), want[r]) for r in range(R) if out[r].item() != want[r]]


@pytest.mark.parametrize("one_cta", [False, True])
def test_sampling_kernel_top_k_and_top_p(ops, one_cta):
    """Few kept candidates are sorted in shared memory; more than 1,024, or top-p alone, are found by selection
    over the whole row. Equal logits are taken in id order; -inf logits weigh nothing. Both kernels: the cluster of
    8 CTAs a row, and the one-CTA kernel of the largest vocabularies."""
    rng = np.random.default_rng(11)
    V = 1531
    rows = []
    for k in (0, 1, 5, 200, 1024, 1100, V, 5000):
        for p in (1.0, 0.9, 0.3, 1e-6):
            rows.append((float(rng.choice([0.3, 0.8, 1.0, 2.5])), k, p, int(rng.integers(0, 2 ** 62))))
    rows += [(0.0, 5, 0.5, 3), (1e-45, 5, 0.5, 3)]                       # greedy whatever the filters say
    R = len(rows)
    z = (rng.standard_normal((R, V)) * 2.5).astype(np.float32)
    z[:, 40:60] = z[:, 700:701]                                          # twenty equal logits in every row
    z[::3, 100:400] = -np.inf
    z[5] = 0.25                                                          # a row of equal logits: the cut falls among ties
    z[6] = np.round(z[6])                                                # many ties at every value
    for counter in (0, 1, 2, 3, 77, 2 ** 33):
        _filtered_case(ops, z, rows, counter, one_cta)
    z[7, 3] = np.inf                                                     # a certain token
    _filtered_case(ops, z, rows, 5, one_cta)


def test_sampling_kernel_filters_over_a_large_vocabulary(ops):
    rng = np.random.default_rng(12)
    V = 151936
    rows = [(0.7, 20, 0.8, 1), (0.7, 0, 0.9, 2), (1.0, 5000, 0.95, 3), (1.3, 0, 0.5, 4), (0.7, 20, 1.0, 5), (1.0, 2000, 1.0, 6)]
    z = (rng.standard_normal((len(rows), V)) * np.array([3, 3, 0.01, 0.01, 5, 1])[:, None]).astype(np.float32)
    for counter in (0, 1, 2):
        _filtered_case(ops, z, rows, counter)
    _filtered_case(ops, z, rows, 3, one_cta=True)


@pytest.mark.parametrize("one_cta", [False, True])
def test_sampling_kernels_refuse_rows_with_a_nan_or_nothing_finite(ops, one_cta):
    """The reference's sampler raises for a NaN logit and for a row of -inf (src/sampling/sampler.cpp:18-26). The
    kernels answer -2 for such a row, with or without filters, and sample the rows beside it as ever."""
    from host_sampler import sample_host
    from tiny_inference_engine_b200.errors import InvalidArgument
    from tiny_inference_engine_b200.sampling import SamplingParams
    rng = np.random.default_rng(21)
    V = 3001
    params = [SamplingParams(temperature=t, top_k=k, top_p=p, seed=7 + i) for i, (t, k, p) in enumerate(
        [(0.0, 0, 1.0), (0.0, 0, 1.0), (0.8, 0, 1.0), (0.8, 0, 1.0), (0.8, 20, 0.9), (0.8, 20, 0.9), (0.8, 20, 0.9),
         (1.0, 0, 0.5), (1.0, 0, 0.5), (0.0, 0, 1.0), (0.7, 5, 1.0)])]
    R = len(params)
    z = (rng.standard_normal((R, V)) * 2).astype(np.float32)
    z[1, 2999] = np.nan          # greedy, a NaN at the far end of the row
    z[3, 0] = np.nan             # temperature, a NaN at the start
    z[5, 1500] = np.nan          # filtered, a NaN in the middle (and a +inf, which does not save the row)
    z[5, 7] = np.inf
    z[6] = -np.inf               # filtered, nothing finite
    z[8] = np.nan                # every logit a NaN
    z[9] = -np.inf               # greedy, nothing finite
    z[10, 5:] = -np.inf          # five finite values left: this row is fine
    refused = {1, 3, 5, 6, 8, 9}
    for r in range(R):
        if r in refused:
            with pytest.raises(InvalidArgument):
                sample_host(z[r], params[r], 3)
    out = torch.full((R,), 77, dtype=torch.int32, device="cuda")
    seeds = np.array([q.seed for q in params], dtype=np.int64)
    ops.sample(dev(z), out, dev(np.array([q.inv_temperature() for q in params], dtype=np.float32)), dev(seeds, torch.int64),
               dev(np.full(R, 3), torch.int64), dev(np.array([q.top_k for q in params]), torch.int32),
               dev(np.array([q.top_p for q in params], dtype=np.float32)), one_cta=one_cta)
    got = out.tolist()
    assert got == [-2 if r in refused else sample_host(z[r], params[r], 3) for r in range(R)]


def test_the_constants_the_host_plans_with_are_the_kernels_own(ops):
    from tiny_inference_engine_b200.ops.library import library
    from tiny_inference_engine_b200.parts import attention as att
    lib = library()
    assert att.TMA_DECODE_TABLE_ENTRIES == lib.tie_attention_decode_limit(0)
    assert att.MAX_SPLITS <= lib.tie_attention_decode_limit(1)
    assert att.NUM_SMS == torch.cuda.get_device_properties(0).multi_processor_count
    assert 1 <= lib.tie_gemm_tc2_pairs() <= att.NUM_SMS // 2


def test_refusals_are_clear(ops):
    from tiny_inference_engine_b200.errors import InvalidArgument
    q = torch.zeros(1, 2 * 20, device="cuda")
    kc = torch.zeros(4, 1, 8, 20, device="cuda")
    i32 = lambda *v: torch.tensor(v, dtype=torch.int32, device="cuda")
    with pytest.raises(InvalidArgument, match="head_dim 20 must be a multiple of 8"):
        ops.attention_rows(q, kc, kc.clone(), torch.zeros_like(q), i32(0), i32(0, 1), i32(1), i32(0, 0).view(1, 2), 2, 1, 20, 1.0)
    with pytest.raises(InvalidArgument, match="not a multiple"):
        ops.attention_rows(torch.zeros(1, 48, device="cuda"), torch.zeros(4, 2, 8, 16, device="cuda"),
                           torch.zeros(4, 2, 8, 16, device="cuda"), torch.zeros(1, 48, device="cuda"), i32(0), i32(0, 1),
                           i32(1), i32(0, 0).view(1, 2), 3, 2, 16, 1.0)
    with pytest.raises(InvalidArgument, match="CUDA tensors"):
        ops.silu_mul(torch.zeros(2, 8), torch.zeros(2, 4))
    with pytest.raises(InvalidArgument, match="shapes"):
        ops.gemm_simt(torch.zeros(2, 8, device="cuda"), torch.zeros(4, 9, device="cuda"), torch.zeros(2, 4, device="cuda"))


@pytest.mark.parametrize("out_dtype", ["bfloat16", "float32"])
@pytest.mark.parametrize("M,N,K", [(1, 503, 96), (3, 311, 144), (8, 1000, 520), (16, 72, 200), (33, 300, 64), (77, 130, 1000),
                                   (128, 256, 512), (200, 96, 72), (300, 503, 96), (700, 311, 136), (513, 256, 64),
                                   (1100, 777, 520)])
def test_gemm_tensor_cores(ops, out_dtype, M, N, K):
    """tcgen05 product with the tiling the engine would pick, at sizes that end inside a tile in
    every direction (rows, columns, k)."""
    from tiny_inference_engine_b200.ops import gemm_select
    rng = np.random.default_rng(M + N + K)
    a, w = as_stored(rng.standard_normal((M, K)), "bfloat16"), as_stored(rng.standard_normal((N, K)), "bfloat16")
    out = torch.full((M, N), float("nan"), device="cuda", dtype=DT[out_dtype])
    ops.gemm(dev(a, torch.bfloat16), dev(w, torch.bfloat16), out)
    torch.cuda.synchronize()
    gemm_select.check_status()
    assert rel_err(host(out), plain.linear(a, w)) < (TOL["bfloat16"] if out_dtype == "bfloat16" else 2e-5)


@pytest.mark.parametrize("M,N,K", [(1, 503, 96), (8, 1000, 520), (16, 72, 200), (77, 130, 1000), (128, 256, 512), (200, 96, 72),
                                   (300, 503, 96), (700, 311, 136), (1100, 2560, 520)])
def test_products_with_the_weight_kept_in_k_blocks(ops, M, N, K):
    """A bound product keeps its weight as [ceil(K / 64), N, 64] (every box a stage loads is one piece of memory) and
    gives the plain product at every token count: the transposed tiling, the 128-token row tiles, the kernel on pairs
    of SMs (the last case), widths and depths that end inside a tile (rows of the next k-block come in with the
    last boxes; they reach no output), a depth that is no multiple of 64 (zeros); and a slice of its rows
    (the k rows of a stacked q/k/v weight) without a copy."""
    from tiny_inference_engine_b200.ops import gemm_select
    rng = np.random.default_rng(M * N + K)
    a, w = as_stored(rng.standard_normal((M, K)), "bfloat16"), as_stored(rng.standard_normal((N, K)), "bfloat16")
    g = ops.bound_gemm(dev(w, torch.bfloat16))
    assert g.packed_rows == N and tuple(g.w.shape) == (-(-K // 64), N, 64) and (g.N, g.K) == (N, K)
    assert torch.equal(g.row_major().cpu(), dev(w, torch.bfloat16).cpu())
    want = plain.linear(a, w)
    for out_dtype in ("bfloat16", "float32"):
        out = torch.full((M, N), float("nan"), device="cuda", dtype=DT[out_dtype])
        got = g(dev(a, torch.bfloat16), out)
        torch.cuda.synchronize()
        gemm_select.check_status()
        assert got is out and rel_err(host(out), want) < (TOL["bfloat16"] if out_dtype == "bfloat16" else 2e-5), out_dtype
    lo, hi = N // 3, N // 3 + max(8, N // 2)
    part = g.rows(lo, hi)
    assert part.w.data_ptr() == g.w.data_ptr() and (part.N, part.row0) == (hi - lo, lo)
    wide = torch.full((M, hi - lo + 16), 7.0, device="cuda", dtype=torch.float32)
    part(dev(a, torch.bfloat16), wide[:, 8:8 + hi - lo])
    torch.cuda.synchronize()
    gemm_select.check_status()
    assert rel_err(host(wide[:, 8:8 + hi - lo]), want[:, lo:hi]) < 2e-5
    assert (wide[:, :8] == 7).all() and (wide[:, 8 + hi - lo:] == 7).all()


@pytest.mark.parametrize("bn", [128, 160, 192, 224, 256])
def test_pair_kernel_at_every_tile_width(ops, bn):
    """The product on pairs of SMs with tiles of 256 rows by 128 to 256 columns, plain and with the SiLU epilogue,
    at sizes that end inside a tile; the width changes which CTA computes what, not what is computed."""
    from tiny_inference_engine_b200.ops import gemm_select
    rng = np.random.default_rng(bn)
    M, N, K = 600, 1000, 264
    a, w = as_stored(rng.standard_normal((M, K)), "bfloat16"), as_stored(rng.standard_normal((N, K)), "bfloat16")
    wide = torch.full((M, N + 16), 7.0, device="cuda", dtype=torch.float32)
    gemm_select.gemm_tc(dev(a, torch.bfloat16), dev(w, torch.bfloat16), wide[:, 8:8 + N], pair=True, bn=bn)
    torch.cuda.synchronize()
    gemm_select.check_status()
    assert rel_err(host(wide[:, 8:8 + N]), plain.linear(a, w)) < 2e-5
    assert (wide[:, :8] == 7).all() and (wide[:, 8 + N:] == 7).all()
    I = 352
    gate, up = as_stored(rng.standard_normal((I, K)) * 0.3, "bfloat16"), as_stored(rng.standard_normal((I, K)) * 0.3, "bfloat16")
    out = torch.full((M, I), float("nan"), device="cuda", dtype=torch.bfloat16)
    gemm_select.gemm_tc(dev(a, torch.bfloat16), ops.interleave_gate_up(dev(gate, torch.bfloat16), dev(up, torch.bfloat16)), out,
                        silu=True, pair=True, bn=bn)
    torch.cuda.synchronize()
    gemm_select.check_status()
    assert rel_err(host(out), plain.swiglu(plain.linear(a, gate), plain.linear(a, up))) < TOL["bfloat16"]


@pytest.mark.parametrize("M", [5, 300, 640])
def test_silu_product_and_split_sums_with_the_weight_in_k_blocks(ops, M):
    from tiny_inference_engine_b200.ops import gemm_select
    rng = np.random.default_rng(M)
    I, K = 352, 264
    a = as_stored(rng.standard_normal((M, K)), "bfloat16")
    gate, up = as_stored(rng.standard_normal((I, K)) * 0.3, "bfloat16"), as_stored(rng.standard_normal((I, K)) * 0.3, "bfloat16")
    g = ops.bound_gemm(ops.interleave_gate_up(dev(gate, torch.bfloat16), dev(up, torch.bfloat16)), silu=True)
    assert g.packed_rows == 2 * I
    out = torch.full((M, I), float("nan"), device="cuda", dtype=torch.bfloat16)
    g(dev(a, torch.bfloat16), out)
    torch.cuda.synchronize()
    gemm_select.check_status()
    assert rel_err(host(out), plain.swiglu(plain.linear(a, gate), plain.linear(a, up))) < TOL["bfloat16"]
    # a split product leaves its partial sums for the consumer, as with a row-major weight
    D, K2 = 520, 4096
    a2, w2 = as_stored(rng.standard_normal((M, K2)), "bfloat16"), as_stored(rng.standard_normal((D, K2)) * 0.05, "bfloat16")
    buf = {}
    got = ops.bound_gemm(dev(w2, torch.bfloat16))(dev(a2, torch.bfloat16), torch.empty(M, D, device="cuda", dtype=torch.bfloat16),
                                                  partial_scratch=lambda n: buf.setdefault("p", torch.full((n,), float("nan"), device="cuda")))
    torch.cuda.synchronize()
    gemm_select.check_status()
    if isinstance(got, ops.SplitSum):
        got = got.materialize(torch.empty(M, D, device="cuda", dtype=torch.float32))
    assert rel_err(host(got), plain.linear(a2, w2)) < TOL["bfloat16"]


def test_embedding_rows_from_a_table_in_k_blocks(ops):
    rng = np.random.default_rng(3)
    V, D = 503, 200                                      # the depth ends inside a k-block
    table = as_stored(rng.standard_normal((V, D)), "bfloat16")
    ids = np.array([0, 502, 17, 17, 256], dtype=np.int32)
    packed = ops.pack_k_blocks(dev(table, torch.bfloat16))
    assert tuple(packed.shape) == (4, V, 64) and torch.equal(ops.unpack_k_blocks(packed, D).cpu(), dev(table, torch.bfloat16).cpu())
    out = torch.full((5, D), float("nan"), device="cuda")
    ops.embed(packed, dev(ids, torch.int32), out)
    assert np.array_equal(host(out), table[ids])


@pytest.mark.parametrize("transposed,bn,splits", [(0, 16, 1), (0, 64, 1), (0, 256, 1), (1, 128, 1), (1, 256, 1), (1, 128, 3),
                                                  (1, 256, 5), (0, 128, 2)])
def test_gemm_tensor_cores_every_tiling(ops, transposed, bn, splits):
    """Every tile width, both orientations, with and without splits of k, into a strided output."""
    from tiny_inference_engine_b200.ops import gemm_select
    rng = np.random.default_rng(bn + splits)
    M, N, K = 77, 300, 520
    a, w = as_stored(rng.standard_normal((M, K)), "bfloat16"), as_stored(rng.standard_normal((N, K)), "bfloat16")
    wide = torch.full((M, N + 40), 7.0, device="cuda", dtype=torch.float32)
    out = wide[:, 8:8 + N]
    gemm_select.gemm_tc(dev(a, torch.bfloat16), dev(w, torch.bfloat16), out, transposed=transposed, bn=bn, splits=splits)
    torch.cuda.synchronize()
    gemm_select.check_status()
    assert rel_err(host(out), plain.linear(a, w)) < 2e-5
    assert (wide[:, :8] == 7).all() and (wide[:, 8 + N:] == 7).all()      # nothing is written beside the output


@pytest.mark.parametrize("bn,splits", [(128, 4), (256, 3), (256, 4)])
def test_gemm_tensor_cores_split_products_of_many_tokens(ops, bn, splits):
    """More tiles times splits than SMs: every split's CTAs walk several tiles, and the sizes end inside a tile in
    every direction. Both the finished product and the partial sums left for a consumer."""
    from tiny_inference_engine_b200.ops import gemm_select
    rng = np.random.default_rng(bn + splits)
    M, N, K = 700, 2000, 1096
    a, w = as_stored(rng.standard_normal((M, K)), "bfloat16"), as_stored(rng.standard_normal((N, K)), "bfloat16")
    want = plain.linear(a, w)
    out = torch.full((M, N), float("nan"), device="cuda", dtype=torch.bfloat16)
    gemm_select.gemm_tc(dev(a, torch.bfloat16), dev(w, torch.bfloat16), out, transposed=0, bn=bn, splits=splits, pair=False)
    torch.cuda.synchronize()
    gemm_select.check_status()
    assert rel_err(host(out), want) < TOL["bfloat16"]
    scratch = torch.full((splits * M * N + 16,), float("nan"), device="cuda")
    got = gemm_select.gemm_tc(dev(a, torch.bfloat16), dev(w, torch.bfloat16), out, transposed=0, bn=bn, splits=splits, pair=False,
                              partial_scratch=lambda n: scratch[:n])
    torch.cuda.synchronize()
    gemm_select.check_status()
    assert isinstance(got, ops.SplitSum) and got.M == M and got.N == N
    parts = scratch[:got.splits * M * N].view(got.splits, M, N)
    assert rel_err(parts.sum(0).cpu().numpy(), want) < 2e-5 and torch.isnan(scratch[got.splits * M * N:]).all()


@pytest.mark.parametrize("silu", [False, True])
def test_gemm_on_pairs_of_sms(ops, silu):
    """The cta_group::2 kernel on more tiles than there are pairs of SMs (each pair walks several,
    alternating its two accumulators), ragged in rows, columns and k, into a strided output; equal,
    bit for bit, to the one-CTA kernel, which adds the same products in the same order."""
    from tiny_inference_engine_b200.ops import gemm_select
    rng = np.random.default_rng(5 + silu)
    M, N, K = 2300, 4000 + 96 * silu, 328
    a = dev(as_stored(rng.standard_normal((M, K)), "bfloat16"), torch.bfloat16)
    w = dev(as_stored(rng.standard_normal((N, K)) * 0.1, "bfloat16"), torch.bfloat16)
    cols = N // 2 if silu else N
    wide = torch.full((M, cols + 24), 7.0, device="cuda", dtype=torch.bfloat16)
    out, want = wide[:, 8:8 + cols], torch.empty(M, cols, device="cuda", dtype=torch.bfloat16)
    for _ in range(2):
        gemm_select.gemm_tc(a, w, out, silu=silu, pair=True)
    gemm_select.gemm_tc(a, w, want, silu=silu, pair=False)
    torch.cuda.synchronize()
    gemm_select.check_status()
    assert torch.equal(out, want)
    assert (wide[:, :8] == 7).all() and (wide[:, 8 + cols:] == 7).all()
    rows = slice(M - 300, M)
    ref = plain.linear(host(a)[rows], host(w))
    if silu:
        ref = ref.reshape(300, -1, 2, 16)
        ref = plain.swiglu(ref[:, :, 0].reshape(300, -1), ref[:, :, 1].reshape(300, -1))
    assert rel_err(host(out)[rows], ref) < TOL["bfloat16"]


def test_gemm_falls_back_when_tma_cannot_address_the_operands(ops):
    """K = 75 is no multiple of 8: the CUDA-core kernel serves it, same numbers."""
    from tiny_inference_engine_b200.ops import gemm_select
    rng = np.random.default_rng(0)
    a, w = as_stored(rng.standard_normal((40, 75)), "bfloat16"), as_stored(rng.standard_normal((90, 75)), "bfloat16")
    ad, wd = dev(a, torch.bfloat16), dev(w, torch.bfloat16)
    out = torch.empty(40, 90, device="cuda", dtype=torch.bfloat16)
    assert not gemm_select.tc_takes(ad, wd, out)
    ops.gemm(ad, wd, out)
    assert rel_err(host(out), plain.linear(a, w)) < TOL["bfloat16"]
    from tiny_inference_engine_b200.errors import InvalidArgument
    with pytest.raises(InvalidArgument, match="multiples of 8"):
        gemm_select.gemm_tc(ad, wd, out)


@pytest.mark.parametrize("Hq,Hkv,Dh,page,window", [(8, 2, 128, 16, 0), (6, 2, 64, 16, 0), (4, 4, 64, 8, 0), (16, 1, 128, 32, 0),
                                                  (3, 1, 256, 16, 0), (8, 2, 128, 16, 100), (5, 5, 64, 4, 37), (32, 2, 64, 64, 0)])
def test_tensor_core_attention_prompt_and_decode(ops, Hq, Hkv, Dh, page, window):
    """The mma kernels on a mixed batch with scattered pages: three sequences bring portions over a
    cached prefix (one of them its whole prompt, one a portion that is no multiple of anything),
    three bring one token with one, two and twelve splits."""
    rng = np.random.default_rng(Hq * Dh + page)
    ctx = [45, 300, 130, 1, 70, 700]
    new = [45, 17, 129, 1, 1, 1]
    kc, vc, bt, ks, vs = paged_cache(rng, "bfloat16", ctx, Hkv, Dh, page, 128 * 16 // page)
    T = sum(new)
    stride = Hq * Dh + 2 * Hkv * Dh                     # q as the engine holds it: the first columns of the qkv rows
    qkv = as_stored(rng.standard_normal((T, stride)), "bfloat16")
    q = qkv[:, :Hq * Dh]
    qs = np.concatenate([[0], np.cumsum(new)])
    scale = 1.0 / np.sqrt(Dh)
    want = np.concatenate([dense_reference(q[qs[i]:qs[i + 1]], ks[i], vs[i], Hq, Hkv, Dh, new[i], window) for i in range(6)])
    qd = dev(qkv, torch.bfloat16)[:, :Hq * Dh]
    assert ops.attention_tc_takes(qd, Hq, Hkv, Dh)
    out = torch.full((T, Hq * Dh), float("nan"), device="cuda", dtype=torch.bfloat16)
    meta = (dev(qs, torch.int32), dev(np.array(ctx), torch.int32), dev(bt, torch.int32))
    n_multi = new[0] + new[1] + new[2]
    ops.attention_prompt_tc(qd, dev(kc, torch.bfloat16), dev(vc, torch.bfloat16), out, *meta, 3, 129, Hq, Hkv, Dh, scale, window)
    assert rel_err(host(out)[:n_multi], want[:n_multi]) < TOL["bfloat16"]
    assert torch.isnan(out[n_multi:].float()).all()          # rows of other sequences are not touched
    if ops.attention_decode_tma_takes(qd, Hq, Hkv, Dh, page):
        from tiny_inference_engine_b200.ops import gemm_select
        out[:] = float("nan")
        ops.attention_prompt_tma(qd, dev(kc, torch.bfloat16), dev(vc, torch.bfloat16), out, *meta, 3, 129, Hq, Hkv, Dh, scale, window)
        torch.cuda.synchronize()
        gemm_select.check_status()
        assert rel_err(host(out)[:n_multi], want[:n_multi]) < TOL["bfloat16"], "TMA-fed prompt kernel"
        assert torch.isnan(out[n_multi:].float()).all()
        if Dh in (64, 128):
            out[:] = float("nan")
            ops.attention_prompt_umma(qd, dev(kc, torch.bfloat16), dev(vc, torch.bfloat16), out, *meta, 3, 129, Hq, Hkv, Dh, scale, window)
            torch.cuda.synchronize()
            gemm_select.check_status()
            assert rel_err(host(out)[:n_multi], want[:n_multi]) < TOL["bfloat16"], "tcgen05 prompt kernel"
            assert torch.isnan(out[n_multi:].float()).all()
    scratch = torch.empty(ops.attention_split_scratch_floats(3, Hq, Dh, 12), device="cuda")
    ops.attention_decode_tc(qd, dev(kc, torch.bfloat16), dev(vc, torch.bfloat16), out, *meta, Hq, Hkv, Dh, scale,
                            dev(np.array([3, 4, 5]), torch.int32), 3, 64, 12, scratch, window)
    assert rel_err(host(out), want) < TOL["bfloat16"]
    # the TMA-fed decode kernel (pages that are powers of two from 8 up), with 1, 2 and many splits, twice
    # in a row so that the second launch finds the counters the first one left
    if ops.attention_decode_tma_takes(qd, Hq, Hkv, Dh, page):
        from tiny_inference_engine_b200.ops import gemm_select
        counters = torch.zeros(3 * Hkv, dtype=torch.int32, device="cuda")
        # and with the splits of a sequence as one cluster that merges through shared memory (2, 4, 8, 16 splits; one
        # of the sequences has a single key, so most of its cluster has nothing to add)
        scratch = torch.empty(ops.attention_split_scratch_floats(3, Hq, Dh, 16), device="cuda")
        for split_keys, max_splits, cluster in ((64, 12, False), (512, 2, False), (1024, 1, False), (64, 12, False), (64, 16, True),
                                                (512, 2, True), (256, 4, True), (128, 8, True), (64, 16, True)):
            out[n_multi:] = float("nan")
            ops.attention_decode_tma(qd, dev(kc, torch.bfloat16), dev(vc, torch.bfloat16), out, *meta, Hq, Hkv, Dh, scale,
                                     3 if cluster else dev(np.array([3, 4, 5]), torch.int32), 3, split_keys, max_splits, scratch,
                                     counters, window, cluster=cluster)
            torch.cuda.synchronize()
            gemm_select.check_status()
            assert rel_err(host(out), want) < TOL["bfloat16"], f"split_keys={split_keys} cluster={cluster}"
            assert not counters.any()


@pytest.mark.parametrize("Hq,Hkv,Dh,page,window", [(8, 2, 128, 16, 0), (4, 4, 64, 8, 0), (16, 1, 128, 32, 0), (6, 2, 256, 16, 0),
                                                  (8, 2, 128, 16, 100), (32, 2, 64, 64, 0)])
@pytest.mark.parametrize("source", ["rows", "partial sums"])
def test_decode_attention_that_prepares_its_own_heads(ops, Hq, Hkv, Dh, page, window, source):
    """A step of single tokens, straight from the q/k/v product's output: the kernel norms and rotates its query
    heads, makes the newest key and value, stores them and uses them. Equal, bit for bit, to the q/k norm + RoPE +
    append kernel followed by the TMA-fed decode attention (outputs and both cache planes; with eight splits the
    kernel under test merges them as a cluster through shared memory, the other through scratch memory), and right against the
    plain attention over keys that include the newest. Contexts that end at the first and the last key of a tile,
    of a page and of a split, one of a single key, one empty (a sequence that pads a captured batch); the newest
    key's slot holds junk before the step, and so do the slots behind it."""
    from tiny_inference_engine_b200.ops import gemm_select
    rng = np.random.default_rng(Hq + Dh + page)
    contexts = [1, 64, 65, 300, 129, 0, 257, 256]
    S = len(contexts)
    kc, vc, bt, ks, vs = paged_cache(rng, "bfloat16", [max(c, 1) for c in contexts], Hkv, Dh, page, 128 * 16 // page)
    width = (Hq + 2 * Hkv) * Dh
    rows = as_stored(rng.standard_normal((S, width)), "bfloat16")
    qw, kw = (1 + 0.2 * rng.standard_normal(Dh)).astype(np.float32), (1 + 0.2 * rng.standard_normal(Dh)).astype(np.float32)
    inv = plain.rope_inv_freq(1e6, Dh)
    pos = np.array([max(c - 1, 0) for c in contexts])
    slots = np.array([bt[i, pos[i] // page] * page + pos[i] % page if contexts[i] > 0 else -1 for i in range(S)])
    for i in range(S):                          # the newest key's slot, and the rest of its page, hold junk
        if contexts[i] > 0:
            kc[bt[i, pos[i] // page], :, pos[i] % page:] = 7.0
            vc[bt[i, pos[i] // page], :, pos[i] % page:] = -7.0
    qs = np.arange(S + 1)
    meta = (dev(qs, torch.int32), dev(np.array(contexts), torch.int32), dev(bt, torch.int32))
    seqs = dev(np.arange(S), torch.int32)
    scale = 1.0 / np.sqrt(Dh)
    partial = None
    if source == "partial sums":                # three float partial sums whose sum, in order, is what the kernels see
        parts = np.stack([rows * 0.5, rows * 0.25, rows * 0.25]).astype(np.float32)
        partial = ops.SplitSum(dev(parts).reshape(-1), 3, S, width)
    results = []
    for fused in (False, True):
        kcd, vcd = dev(kc, torch.bfloat16), dev(vc, torch.bfloat16)
        qkv = dev(rows if partial is None else np.zeros_like(rows), torch.bfloat16)
        out = torch.full((S, Hq * Dh), float("nan"), device="cuda", dtype=torch.bfloat16)
        scratch = torch.empty(ops.attention_split_scratch_floats(S, Hq, Dh, 8), device="cuda")
        counters = torch.zeros(S * Hkv, dtype=torch.int32, device="cuda")
        for split_keys, max_splits in ((64, 8), (128, 3), (512, 1)):
            if fused:
                assert ops.attention_decode_prep_takes(qkv, Hq, Hkv, Dh, page, dev(inv))
                # (the sequences as "S in a row from 0 on" instead of a list, for every other split size)
                ops.attention_decode_prep(qkv, dev(qw), dev(kw), 1e-6, 1e-5, dev(inv), dev(pos, torch.int32), kcd, vcd, out, *meta,
                                          Hq, Hkv, Dh, scale, 0 if split_keys != 128 else seqs, S, split_keys, max_splits, scratch,
                                          counters, window, append=True, partial=partial, cluster=max_splits in ops.CLUSTER_SPLITS)
            else:
                work = qkv.clone()
                ops.qk_norm_rope_append(work, dev(qw), dev(kw), 1e-6, 1e-5, dev(inv), dev(pos, torch.int32), dev(slots, torch.int32),
                                        kcd, vcd, Hq, Hkv, Dh, partial=partial)
                ops.attention_decode_tma(work[:, :Hq * Dh], kcd, vcd, out, *meta, Hq, Hkv, Dh, scale, seqs, S, split_keys,
                                         max_splits, scratch, counters, window)
            torch.cuda.synchronize()
            gemm_select.check_status()
            assert not counters.any()
            results.append((fused, split_keys, out.clone(), kcd.clone(), vcd.clone()))
    half = len(results) // 2
    for (_, sk, o0, k0, v0), (_, _, o1, k1, v1) in zip(results[:half], results[half:]):
        assert torch.equal(o0, o1), f"outputs differ at split_keys={sk}"
        assert torch.equal(k0, k1) and torch.equal(v0, v1), "cache planes differ"
    # against the plain formulas: the newest key and value are among the keys
    q, k, v = rows[:, :Hq * Dh], rows[:, Hq * Dh:(Hq + Hkv) * Dh], rows[:, (Hq + Hkv) * Dh:]
    want_q = as_stored(plain.rope_neox(plain.rms_norm(q.reshape(S * Hq, Dh), qw, 1e-6).reshape(S, -1), pos, Hq, Dh, 1e6), "bfloat16")
    want_k = as_stored(plain.rope_neox(plain.rms_norm(k.reshape(S * Hkv, Dh), kw, 1e-5).reshape(S, -1), pos, Hkv, Dh, 1e6), "bfloat16")
    got = host(results[-1][2])
    for i, c in enumerate(contexts):
        if c == 0:
            assert not got[i].any()
            continue
        keys = np.concatenate([ks[i][:c - 1], want_k[i].reshape(1, Hkv, Dh)])
        vals = np.concatenate([vs[i][:c - 1], v[i].reshape(1, Hkv, Dh)])
        want = dense_reference(want_q[i:i + 1], keys, vals, Hq, Hkv, Dh, 1, window)
        assert rel_err(got[i:i + 1], want) < TOL["bfloat16"], f"context {c}"
    # without the append (a layer that reads another layer's cache): the cache is read as it is and left as it is
    kcd, vcd = results[4][3].clone(), results[4][4].clone()     # the planes as the run with 3 splits of 128 keys left them
    before_k, before_v = kcd.clone(), vcd.clone()
    out = torch.full((S, Hq * Dh), float("nan"), device="cuda", dtype=torch.bfloat16)
    q_only = dev(rows, torch.bfloat16)[:, :Hq * Dh]
    ops.attention_decode_prep(q_only, dev(qw), dev(kw), 1e-6, 1e-5, dev(inv), dev(pos, torch.int32), kcd, vcd, out, *meta,
                              Hq, Hkv, Dh, scale, seqs, S, 128, 3, scratch, counters, window, append=False)
    torch.cuda.synchronize()
    gemm_select.check_status()
    assert torch.equal(kcd, before_k) and torch.equal(vcd, before_v)
    if partial is None:
        assert torch.equal(out, results[4][2])


@pytest.mark.parametrize("far", [0, 15, 16, 63, 64, 65, 255, 256, 511, 512, 1022, 1023])
def test_tensor_core_attention_finds_one_far_key(ops, far):
    """As test_one_far_key_among_a_thousand_is_found, for the mma kernels: edges of pages (16),
    of a warp's 16 keys, of 64-key tiles, of 256-key splits, the first and the last key."""
    rng = np.random.default_rng(far)
    Hq, Hkv, Dh, page, n = 8, 2, 64, 16, 1024
    kc, vc, bt, ks, vs = paged_cache(rng, "bfloat16", [n, n], Hkv, Dh, page, 140)
    for n_new in (1, 40):                                  # decode kernel, then the prompt kernel (last 40 rows)
        q = np.zeros((n_new, Hq * Dh), dtype=np.float32)
        for h in range(Hq):
            q[-1, h * Dh:(h + 1) * Dh] = 8.0 * ks[0][far, h // 4] * np.sqrt(Dh)
        q = as_stored(q, "bfloat16")
        want = dense_reference(q, ks[0], vs[0], Hq, Hkv, Dh, n_new)
        one_hot = np.concatenate([vs[0][far, h // 4] for h in range(Hq)])
        if far <= n - n_new or n_new == 1:
            assert np.abs(want[-1] - one_hot).max() < 2e-3
        meta = (dev(np.array([0, n_new]), torch.int32), dev(np.array([n]), torch.int32), dev(bt[:1], torch.int32))
        out = torch.zeros(n_new, Hq * Dh, device="cuda", dtype=torch.bfloat16)
        args = (dev(q, torch.bfloat16), dev(kc, torch.bfloat16), dev(vc, torch.bfloat16), out)
        if n_new == 1:
            scratch = torch.empty(ops.attention_split_scratch_floats(1, Hq, Dh, 4), device="cuda")
            ops.attention_decode_tc(*args, *meta, Hq, Hkv, Dh, 1 / np.sqrt(Dh), dev(np.array([0]), torch.int32), 1, 256, 4, scratch)
            assert np.abs(host(out)[-1] - want[-1]).max() < 2e-2, "cp.async decode kernel"
            out.zero_()
            ops.attention_decode_tma(*args, *meta, Hq, Hkv, Dh, 1 / np.sqrt(Dh), dev(np.array([0]), torch.int32), 1, 256, 4,
                                     scratch, torch.zeros(Hkv, dtype=torch.int32, device="cuda"))
        else:
            ops.attention_prompt_tc(*args, *meta, 1, n_new, Hq, Hkv, Dh, 1 / np.sqrt(Dh))
            assert np.abs(host(out)[-1] - want[-1]).max() < 2e-2, "cp.async prompt kernel"
            out.zero_()
            ops.attention_prompt_tma(*args, *meta, 1, n_new, Hq, Hkv, Dh, 1 / np.sqrt(Dh))
            assert np.abs(host(out)[-1] - want[-1]).max() < 2e-2, "TMA-fed prompt kernel"
            out.zero_()
            ops.attention_prompt_umma(*args, *meta, 1, n_new, Hq, Hkv, Dh, 1 / np.sqrt(Dh))
        assert np.abs(host(out)[-1] - want[-1]).max() < 2e-2, f"n_new={n_new}"


@pytest.mark.parametrize("Hq,Hkv,Dh,page,window", [(8, 2, 128, 16, 0), (6, 2, 64, 8, 0), (3, 3, 128, 64, 0), (16, 1, 64, 128, 0),
                                                  (8, 2, 128, 16, 70), (10, 2, 64, 32, 333), (32, 2, 128, 16, 0), (32, 2, 128, 16, 100)])
def test_tcgen05_prompt_attention_on_long_portions(ops, Hq, Hkv, Dh, page, window):
    """Portions that fill several 256-row tiles and end inside one: a whole prompt, a portion over a long
    cached prefix, a portion whose rows end one short of a tile, and a short one; scattered pages. With 16 query
    heads to a key head there are so many rows that a CTA takes two row tiles; with fewer, one."""
    from tiny_inference_engine_b200.ops import gemm_select
    rng = np.random.default_rng(Hq + Dh + page + window)
    ctx = [333, 900, 64 * 3 - 1, 21]
    new = [333, 257, 64 * 3 - 1, 5]
    kc, vc, bt, ks, vs = paged_cache(rng, "bfloat16", ctx, Hkv, Dh, page, sum(-(-c // page) for c in ctx) + 5)
    T = sum(new)
    qkv = as_stored(rng.standard_normal((T, Hq * Dh + 2 * Hkv * Dh)), "bfloat16")
    q = qkv[:, :Hq * Dh]
    qs = np.concatenate([[0], np.cumsum(new)])
    want = np.concatenate([dense_reference(q[qs[i]:qs[i + 1]], ks[i], vs[i], Hq, Hkv, Dh, new[i], window) for i in range(4)])
    qd = dev(qkv, torch.bfloat16)[:, :Hq * Dh]
    out = torch.full((T + 3, Hq * Dh), float("nan"), device="cuda", dtype=torch.bfloat16)
    meta = (dev(qs, torch.int32), dev(np.array(ctx), torch.int32), dev(bt, torch.int32))
    assert ops.attention_prompt_umma_takes(qd, Hq, Hkv, Dh, page, max(new))
    for _ in range(2):
        ops.attention_prompt_umma(qd, dev(kc, torch.bfloat16), dev(vc, torch.bfloat16), out[:T], *meta, 4, max(new), Hq, Hkv, Dh,
                                  1 / np.sqrt(Dh), window)
    torch.cuda.synchronize()
    gemm_select.check_status()
    assert rel_err(host(out)[:T], want) < TOL["bfloat16"]
    assert torch.isnan(out[T:].float()).all()


def test_tcgen05_prompt_attention_when_the_maximum_keeps_growing(ops):
    """Scores that rise along the keys by about 3 (in powers of two) a key: every tile moves the
    reference point of the exponentials, so the accumulator in tensor memory is rescaled again and again;
    and scores that fall, so that it never is after the first tile."""
    from tiny_inference_engine_b200.ops import gemm_select
    rng = np.random.default_rng(11)
    Hq, Hkv, Dh, page, n = 4, 1, 64, 16, 640
    for rising in (True, False):
        kc, vc, bt, ks, vs = paged_cache(rng, "bfloat16", [n], Hkv, Dh, page, 48)
        u = rng.standard_normal(Dh)
        u /= np.linalg.norm(u)
        ramp = np.arange(n) if rising else n - np.arange(n)
        keys = as_stored(ramp[:, None] * u[None, :] * 0.25 + 0.05 * rng.standard_normal((n, Dh)), "bfloat16")
        for t in range(n):                                  # overwrite the cached keys in their pages
            kc[bt[0, t // page], 0, t % page] = keys[t]
        q = as_stored(np.tile(u * 8.0 * np.sqrt(Dh) * np.log(2), (n, Hq)) + 0.1 * rng.standard_normal((n, Hq * Dh)), "bfloat16")
        want = dense_reference(q, keys.reshape(n, Hkv, Dh), vs[0], Hq, Hkv, Dh, n)
        out = torch.zeros(n, Hq * Dh, device="cuda", dtype=torch.bfloat16)
        ops.attention_prompt_umma(dev(q, torch.bfloat16), dev(kc, torch.bfloat16), dev(vc, torch.bfloat16), out,
                                  dev(np.array([0, n]), torch.int32), dev(np.array([n]), torch.int32), dev(bt, torch.int32), 1, n,
                                  Hq, Hkv, Dh, 1 / np.sqrt(Dh))
        torch.cuda.synchronize()
        gemm_select.check_status()
        assert rel_err(host(out), want) < TOL["bfloat16"], f"rising={rising}"


@pytest.mark.parametrize("page,longest", [(8, 4500), (16, 8300)])
def test_decode_attention_over_long_contexts_with_the_longest_splits(ops, page, longest):
    """Contexts beyond what one split may hold (the kernel keeps a split's page ids in shared memory): the part's
    choice of split size stays inside the limit and the result is the dense one."""
    from tiny_inference_engine_b200.ops import gemm_select
    from tiny_inference_engine_b200.parts.attention import decode_splits
    rng = np.random.default_rng(page)
    Hq, Hkv, Dh = 4, 2, 64
    split_keys, max_splits = decode_splits(longest, 200, Hkv, page)       # so many sequences that each gets one CTA per kv head
    assert max_splits == 2 and split_keys < longest
    ctx = [longest, split_keys + 1, split_keys, 10, 1]
    kc, vc, bt, ks, vs = paged_cache(rng, "bfloat16", ctx, Hkv, Dh, page, sum(-(-c // page) for c in ctx) + 3)
    S = len(ctx)
    q = as_stored(rng.standard_normal((S, Hq * Dh)), "bfloat16")
    want = np.concatenate([dense_reference(q[i:i + 1], ks[i], vs[i], Hq, Hkv, Dh, 1) for i in range(S)])
    out = torch.full((S, Hq * Dh), float("nan"), device="cuda", dtype=torch.bfloat16)
    scratch = torch.empty(ops.attention_split_scratch_floats(S, Hq, Dh, max_splits), device="cuda")
    counters = torch.zeros(S * Hkv, dtype=torch.int32, device="cuda")
    ops.attention_decode_tma(dev(q, torch.bfloat16), dev(kc, torch.bfloat16), dev(vc, torch.bfloat16), out,
                             dev(np.arange(S + 1), torch.int32), dev(np.array(ctx), torch.int32), dev(bt, torch.int32), Hq, Hkv, Dh,
                             1 / np.sqrt(Dh), dev(np.arange(S), torch.int32), S, split_keys, max_splits, scratch, counters)
    torch.cuda.synchronize()
    gemm_select.check_status()
    assert rel_err(host(out), want) < TOL["bfloat16"] and not counters.any()


def test_a_context_beyond_the_splits_a_call_allows_costs_time_or_is_refused_but_never_keys(ops):
    """A caller of the exported kernels who sizes max_splits from something else than the longest context: the
    CUDA-core and cp.async kernels let the last split take the rest (the merge reads no more splits than there
    are), the TMA kernel, whose splits are bounded by its page table in shared memory, says so in the status word."""
    from tiny_inference_engine_b200.errors import TieError
    from tiny_inference_engine_b200.ops import gemm_select
    rng = np.random.default_rng(77)
    Hq, Hkv, Dh, page = 4, 2, 64, 16
    ctx = [700, 130, 64, 1]                      # 700 keys need 6 splits of 128; the call allows 2
    split_keys, max_splits, S = 128, 2, len(ctx)
    for dtype in ("float32", "bfloat16"):
        kc, vc, bt, ks, vs = paged_cache(rng, dtype, ctx, Hkv, Dh, page, sum(-(-c // page) for c in ctx) + 3)
        q = as_stored(rng.standard_normal((S, Hq * Dh)), dtype)
        want = np.concatenate([dense_reference(q[i:i + 1], ks[i], vs[i], Hq, Hkv, Dh, 1) for i in range(S)])
        args = (dev(np.arange(S + 1), torch.int32), dev(np.array(ctx), torch.int32), dev(bt, torch.int32), Hq, Hkv, Dh,
                1 / np.sqrt(Dh), dev(np.arange(S), torch.int32), S, split_keys, max_splits)
        fns = [ops.attention_split] + ([ops.attention_decode_tc] if dtype == "bfloat16" else [])
        for fn in fns:
            out = torch.full((S, Hq * Dh), float("nan"), device="cuda", dtype=DT[dtype])
            scratch = torch.full((ops.attention_split_scratch_floats(S, Hq, Dh, max_splits),), float("nan"), device="cuda")
            fn(dev(q, DT[dtype]), dev(kc, DT[dtype]), dev(vc, DT[dtype]), out, *args, scratch)
            torch.cuda.synchronize()
            assert rel_err(host(out), want) < TOL[dtype], fn.__name__
    out = torch.full((S, Hq * Dh), float("nan"), device="cuda", dtype=torch.bfloat16)
    counters = torch.zeros(S * Hkv, dtype=torch.int32, device="cuda")
    ops.attention_decode_tma(dev(q, torch.bfloat16), dev(kc, torch.bfloat16), dev(vc, torch.bfloat16), out, *args, scratch, counters)
    torch.cuda.synchronize()
    with pytest.raises(TieError, match="fewer splits"):
        gemm_select.check_status()
    assert torch.isnan(out[0].float()).all() and rel_err(host(out)[1:], want[1:]) < TOL["bfloat16"]
    gemm_select.check_status()                   # read and cleared


def test_tensor_core_attention_refuses_other_sizes(ops):
    q = torch.zeros(4, 2 * 48, device="cuda", dtype=torch.bfloat16)
    assert not ops.attention_tc_takes(q, 2, 1, 48)
    assert not ops.attention_tc_takes(torch.zeros(4, 34 * 64, device="cuda", dtype=torch.bfloat16), 34, 2, 64)
    assert not ops.attention_tc_takes(torch.zeros(4, 128, device="cuda"), 2, 1, 64)


@pytest.mark.parametrize("M", [100, 200, 300])
def test_split_products_of_many_tokens_feed_the_norm(ops, M):
    """Between 65 and a few hundred tokens a product with few output tiles cuts k as well (128-token row
    tiles, or the weights on the 128-row side up to 128 tokens): the partial sums reach the add+norm
    kernel as they are."""
    from tiny_inference_engine_b200.ops import gemm_select
    rng = np.random.default_rng(M)
    D, K = 520, 4096
    transposed, bn, splits = gemm_select.plan(M, D, K)
    assert splits > 1 and transposed == (M <= 128)
    a, w = as_stored(rng.standard_normal((M, K)), "bfloat16"), as_stored(rng.standard_normal((D, K)) * 0.05, "bfloat16")
    buf = {}
    got = ops.gemm(dev(a, torch.bfloat16), dev(w, torch.bfloat16), torch.empty(M, D, device="cuda", dtype=torch.bfloat16),
                   partial_scratch=lambda n: buf.setdefault("p", torch.full((n,), float("nan"), device="cuda")))
    assert isinstance(got, ops.SplitSum) and 1 < got.splits <= splits and (got.M, got.N) == (M, D)
    prod = plain.linear(a, w)
    x = rng.standard_normal((M, D)).astype(np.float32)
    wn = (1 + 0.1 * rng.standard_normal(D)).astype(np.float32)
    xd, out = dev(x), torch.empty(M, D, device="cuda", dtype=torch.bfloat16)
    ops.add_rmsnorm(xd, got, dev(wn), 1e-6, out)
    torch.cuda.synchronize()
    gemm_select.check_status()
    assert np.abs(host(xd) - (x + prod)).max() < 1e-4 * np.abs(prod).max()
    assert rel_err(host(out), plain.rms_norm(x + prod, wn, 1e-6)) < TOL["bfloat16"]


def test_split_products_hand_partial_sums_to_their_consumers(ops):
    """A decode-sized product whose k range is cut leaves float partial sums; the add+norm kernel and
    the q/k norm + RoPE + append kernel add them up themselves. Same numbers as the unsplit way."""
    rng = np.random.default_rng(3)
    M, D, K = 5, 1024, 2048
    a, w = as_stored(rng.standard_normal((M, K)), "bfloat16"), as_stored(rng.standard_normal((D, K)) * 0.05, "bfloat16")
    bufs = {}
    got = ops.gemm(dev(a, torch.bfloat16), dev(w, torch.bfloat16), torch.empty(M, D, device="cuda", dtype=torch.bfloat16),
                   partial_scratch=lambda n: bufs.setdefault("p", torch.empty(n, device="cuda")))
    assert isinstance(got, ops.SplitSum) and got.splits > 1 and (got.M, got.N) == (M, D)
    prod = plain.linear(a, w)
    whole = got.materialize(torch.empty(M, D, device="cuda"))
    assert rel_err(host(whole), prod) < 2e-5
    # residual add + norm straight from the partial sums
    x = rng.standard_normal((M, D)).astype(np.float32)
    wn = (1 + 0.1 * rng.standard_normal(D)).astype(np.float32)
    xd, out = dev(x), torch.empty(M, D, device="cuda", dtype=torch.bfloat16)
    ops.add_rmsnorm(xd, got, dev(wn), 1e-6, out)
    assert np.abs(host(xd) - (x + prod)).max() < 1e-4 * np.abs(prod).max()
    assert rel_err(host(out), plain.rms_norm(x + prod, wn, 1e-6)) < TOL["bfloat16"]
    rows = np.array([4, 1])
    out2, x2 = torch.empty(2, D, device="cuda", dtype=torch.bfloat16), dev(x)
    ops.add_rmsnorm(x2, got, dev(wn), 1e-6, out2, rows=dev(rows, torch.int32))
    assert np.array_equal(host(x2), x) and rel_err(host(out2), plain.rms_norm((x + prod)[rows], wn, 1e-6)) < TOL["bfloat16"]
    # q/k norm + RoPE + append from the partial sums of a q,k,v product
    Hq, Hkv, Dh, page = 4, 2, 128, 16
    width = (Hq + 2 * Hkv) * Dh
    wq = as_stored(rng.standard_normal((width, K)) * 0.05, "bfloat16")
    qkv = torch.zeros(M, width, device="cuda", dtype=torch.bfloat16)
    ps = ops.gemm(dev(a, torch.bfloat16), dev(wq, torch.bfloat16), qkv,
                  partial_scratch=lambda n: bufs.setdefault("q", torch.empty(n, device="cuda")))
    assert isinstance(ps, ops.SplitSum)
    full = plain.linear(a, wq)
    qw, kw = (1 + 0.2 * rng.standard_normal(Dh)).astype(np.float32), (1 + 0.2 * rng.standard_normal(Dh)).astype(np.float32)
    pos, slots = np.array([0, 5, 77, 1000, 3]), np.array([3, 17, 40, -1, 8])
    kc, vc = torch.zeros(4, Hkv, page, Dh, device="cuda", dtype=torch.bfloat16), torch.zeros(4, Hkv, page, Dh, device="cuda", dtype=torch.bfloat16)
    ops.qk_norm_rope_append(qkv, dev(qw), dev(kw), 1e-6, 1e-6, dev(plain.rope_inv_freq(1e6, Dh)), dev(pos, torch.int32),
                            dev(slots, torch.int32), kc, vc, Hq, Hkv, Dh, partial=ps)
    q, k, v = full[:, :Hq * Dh], full[:, Hq * Dh:(Hq + Hkv) * Dh], full[:, (Hq + Hkv) * Dh:]
    want_q = plain.rope_neox(plain.rms_norm(q.reshape(M * Hq, Dh), qw, 1e-6).reshape(M, -1), pos, Hq, Dh, 1e6)
    want_k = plain.rope_neox(plain.rms_norm(k.reshape(M * Hkv, Dh), kw, 1e-6).reshape(M, -1), pos, Hkv, Dh, 1e6)
    assert rel_err(host(qkv)[:, :Hq * Dh], want_q) < TOL["bfloat16"]
    for t in range(M):
        if slots[t] >= 0:
            p, o = slots[t] // page, slots[t] % page
            assert rel_err(host(kc)[p, :, o].reshape(1, -1), want_k[t].reshape(1, -1)) < TOL["bfloat16"]
            assert rel_err(host(vc)[p, :, o].reshape(1, -1), v[t].reshape(1, -1)) < TOL["bfloat16"]


@pytest.mark.parametrize("M", [1, 7, 64, 200, 300, 700])
@pytest.mark.parametrize("I,K", [(16, 64), (48, 72), (208, 136), (1536, 1024)])
def test_gemm_with_silu_epilogue(ops, M, I, K):
    """silu(a gate^T) * (a up^T) in the product's epilogue, both tilings, widths that end inside a tile."""
    rng = np.random.default_rng(M + I)
    a = as_stored(rng.standard_normal((M, K)), "bfloat16")
    gate, up = as_stored(rng.standard_normal((I, K)) * 0.2, "bfloat16"), as_stored(rng.standard_normal((I, K)) * 0.2, "bfloat16")
    w = ops.interleave_gate_up(dev(gate, torch.bfloat16), dev(up, torch.bfloat16))
    assert np.array_equal(host(w)[:16], gate[:16]) and np.array_equal(host(w)[16:32], up[:16])
    out = torch.full((M, I), float("nan"), device="cuda", dtype=torch.bfloat16)
    ops.gemm_silu(dev(a, torch.bfloat16), w, out)
    assert rel_err(host(out), plain.swiglu(plain.linear(a, gate), plain.linear(a, up))) < TOL["bfloat16"]
