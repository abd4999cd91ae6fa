"""Parity of each CUDA kernel, called through the C boundary, against the CPU oracle on the
same seeded inputs. Integer / byte results are compared bit for bit; floating-point ones
within the tolerances written at each test (the path's stated bar is 2e-3 on logits)."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from oracle import oracle  # noqa: E402
from tests.workloads import WideDecodeCase, c2_contexts, paged_attention_case, round_f16  # noqa: E402


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.fail("the gpu tests need a CUDA device")
    from relay_b200 import ops as o
    return o


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


def row_err(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    a, b = a.reshape(a.shape[0], -1), b.reshape(b.shape[0], -1)
    return float((np.abs(a - b).max(1) / np.maximum(np.abs(b).max(1), 1e-6)).max())


# ---- small kernels -------------------------------------------------------------------------

def test_f32_to_f16_is_bit_exact(ops):
    z = np.load("tests/golden/f16_known_answers.npz")
    x = z["f32_in"]
    out = torch.empty(x.size, dtype=torch.float16, device="cuda")
    ops.f32_to_f16(dev(x), out)
    got = out.cpu().numpy().view(np.uint16)
    nan = np.isnan(x)
    assert np.array_equal(got[~nan], z["f16_bits"][~nan])
    assert np.all(np.isnan(out.cpu().numpy()[nan]))


@pytest.mark.parametrize("H,ld", [(64, 64), (172, 192), (4096, 4096), (1000, 1024)])
def test_rmsnorm(ops, H, ld):
    rng = np.random.Generator(np.random.PCG64(1))
    x = rng.standard_normal((7, H)).astype(np.float32) * 3
    w = (1 + 0.1 * rng.standard_normal(H)).astype(np.float32)
    rows = np.asarray([6, 0, 3], np.int32)
    want = oracle.rmsnorm(x, w, 1e-5)
    out = torch.full((7, ld), 9.0, dtype=torch.float16, device="cuda")
    ops.rmsnorm(dev(x), dev(w), out, 1e-5)
    got = out.cpu().numpy().astype(np.float32)
    assert np.abs(got[:, :H] - want).max() <= 1e-3 * np.abs(want).max() + 1e-6  # fp16 output rounding: 2^-11 relative
    assert np.all(got[:, H:] == 0)
    out2 = torch.empty((3, ld), dtype=torch.float16, device="cuda")
    ops.rmsnorm(dev(x), dev(w), out2, 1e-5, rows=dev(rows))
    assert torch.equal(out2, out[torch.from_numpy(rows).long().cuda()])


def test_embed_and_silu_mul(ops):
    rng = np.random.Generator(np.random.PCG64(2))
    table = round_f16(rng.standard_normal((50, 72)))
    toks = np.asarray([3, 49, 0, 3], np.int32)
    x = torch.empty((4, 72), dtype=torch.float32, device="cuda")
    ops.embed(dev(toks), dev(table, torch.float16), x)
    assert np.array_equal(x.cpu().numpy(), table[toks])
    for I, ld in [(172, 192), (160, 160), (14336, 14336)]:
        gu = (rng.standard_normal((5, 2 * I)) * 2).astype(np.float32)
        want = oracle.swiglu(gu)
        act = torch.full((5, ld), 7.0, dtype=torch.float16, device="cuda")
        ops.silu_mul(dev(gu), act)
        got = act.cpu().numpy().astype(np.float32)
        assert np.abs(got[:, :I] - want).max() <= 1e-3 * np.abs(want).max()
        assert np.all(got[:, I:] == 0)


@pytest.mark.parametrize("D,heads,kv_heads,bs,llama3", [(16, 4, 2, 16, False), (128, 32, 8, 16, True), (64, 8, 8, 1, False), (8, 8, 2, 32, False)])
def test_qkv_post_rope_and_kv_append(ops, D, heads, kv_heads, bs, llama3):
    from relay_b200.types import ModelConfig
    rng = np.random.Generator(np.random.PCG64(3))
    cfg = ModelConfig(hidden=64, intermediate=64, layers=1, heads=heads, kv_heads=kv_heads, head_dim=D, vocab=8,
                      rope_theta=500000.0 if llama3 else 10000.0, rope_scaling_type="llama3" if llama3 else "",
                      rope_factor=8.0, rope_original_max_position=8192.0)
    inv = oracle.rope_inv_freq(cfg)
    nb = 300
    # three sequences: a 19-token chunk starting at 5, a decode token at 4000 (large angles), one at 0
    chunks = [(5, 19), (4000 if bs >= 16 else 37, 1), (0, 1)]
    pos, seq, toff, tables = [], [], [], []
    cursor = 0
    for s, (p0, n) in enumerate(chunks):
        toff.append(len(tables))
        for _ in range((p0 + n + bs - 1) // bs):
            tables.append(int((cursor * 7 + 3) % nb))  # 7 is coprime with 300: every block id is distinct
            cursor += 1
        pos += list(range(p0, p0 + n))
        seq += [s] * n
    T = len(pos)
    QKV = (heads + 2 * kv_heads) * D
    qkv = rng.standard_normal((T, QKV)).astype(np.float32)
    bias = (0.1 * rng.standard_normal(QKV)).astype(np.float32)
    pos, seq, toff, tables = (np.asarray(a, np.int32) for a in (pos, seq, toff, tables))
    for use_bias in (False, True):
        want_qkv = qkv.copy()
        kp = np.zeros((nb, kv_heads, bs, D), np.float32)
        vp = np.zeros_like(kp)
        oracle.qkv_post(want_qkv, bias if use_bias else None, inv, pos, seq, toff, tables, kp, vp, heads, kv_heads, D, bs)
        g_qkv = dev(qkv)
        g_k = torch.zeros((nb, kv_heads, bs, D), dtype=torch.float16, device="cuda")
        g_v = torch.zeros_like(g_k)
        meta = ops.TokenMeta.from_host(pos, seq, toff, tables)
        ops.qkv_post(g_qkv, dev(bias) if use_bias else None, dev(inv), meta, g_k, g_v, heads, kv_heads, D, bs)
        got = g_qkv.cpu().numpy()
        # q and k rotated in fp32: sin/cos differ from the host's by a few ulp at most
        assert np.abs(got - want_qkv).max() <= 4e-6 * max(1.0, np.abs(want_qkv).max())
        # pages: the fp16 rounding of the fp32 values, up to one fp16 step where the fp32 inputs differ by an ulp
        for gp, wp in ((g_k, kp), (g_v, vp)):
            g16 = gp.cpu().numpy()
            w16 = wp.astype(np.float16)
            steps = np.abs(g16.view(np.int16).astype(np.int32) - w16.view(np.int16).astype(np.int32))
            assert steps.max() <= 1 and (steps > 0).mean() < 2e-3
            assert np.array_equal(g16 == 0, w16 == 0)  # untouched slots stay zero, written ones are written
        # V is copied, not rotated: bit-exact
        assert np.array_equal(g_v.cpu().numpy().view(np.uint16), vp.astype(np.float16).view(np.uint16))


def test_kv_gather_scatter_are_byte_exact(ops):
    rng = np.random.Generator(np.random.PCG64(4))
    bb, nb = 32768, 24
    k = rng.integers(0, 256, nb * bb, dtype=np.uint8)
    v = rng.integers(0, 256, nb * bb, dtype=np.uint8)
    blocks = np.asarray([7, 2, 23, 0, 11], np.int32)
    st = torch.empty(2 * blocks.size * bb, dtype=torch.uint8, device="cuda")
    ops.kv_gather(dev(k), dev(v), dev(blocks), bb, st)
    assert np.array_equal(st.cpu().numpy(), oracle.kv_gather(k, v, blocks, bb))
    k2, v2 = torch.zeros(nb * bb, dtype=torch.uint8, device="cuda"), torch.zeros(nb * bb, dtype=torch.uint8, device="cuda")
    dst = np.asarray([1, 5, 4, 22, 9], np.int32)
    ops.kv_scatter(k2, v2, dev(dst), bb, st)
    wk, wv = np.zeros_like(k), np.zeros_like(v)
    oracle.kv_scatter(wk, wv, dst, bb, st.cpu().numpy())
    assert np.array_equal(k2.cpu().numpy(), wk) and np.array_equal(v2.cpu().numpy(), wv)


def test_argmax_rows_lowest_id_wins_ties(ops):
    rng = np.random.Generator(np.random.PCG64(5))
    lg = rng.standard_normal((9, 128256)).astype(np.float32)
    lg[0, [77, 9000, 100000]] = 50.0
    lg[1, :] = 0.0
    lg[2, 128255] = 60.0
    tok = torch.empty(9, dtype=torch.int32, device="cuda")
    val = torch.empty(9, dtype=torch.float32, device="cuda")
    ops.argmax_rows(dev(lg), tok, val)
    want = [oracle.argmax(r) for r in lg]
    assert tok.cpu().tolist() == want and want[0] == 77 and want[1] == 0
    assert np.array_equal(val.cpu().numpy(), lg[np.arange(9), want])


# ---- attention -------------------------------------------------------------------------------

def run_attention(ops, case, kind):
    c = case
    heads, kv_heads, D, bs = c["heads"], c["kv_heads"], c["D"], c["bs"]
    T = len(c["pos"])
    shape = ops.attn_shape(heads, kv_heads, D, bs)
    meta = ops.TokenMeta.from_host(c["pos"], c["seq"], c["table_off"], c["tables"])
    q = dev(c["q"])
    kp, vp = dev(c["k_pool"], torch.float16), dev(c["v_pool"], torch.float16)
    out = torch.zeros((T, heads * D), dtype=torch.float16, device="cuda")
    if kind == "decode":
        toks = dev(np.arange(T, dtype=np.int32))
        ops.decode_attention(shape, q, meta, toks, int(max(c["ctxs"])), kp, vp, out)
    elif kind == "prefill":
        tiles, t = [], 0
        for n in c["chunk_lens"]:
            for r in range(0, n, 64):
                tiles += [t + r, min(64, n - r)]
            t += n
        ops.prefill_attention(shape, q, meta, dev(np.asarray(tiles, np.int32)), kp, vp, out)
    else:
        ops.reference_attention(shape, q, meta, T, kp, vp, out)
    torch.cuda.synchronize()
    assert ops.gemm_status() == 0  # no bounded pipeline wait of a tcgen05 kernel gave up
    return out.cpu().numpy().astype(np.float32)


def oracle_attention(c):
    return oracle.attention(c["q"], c["q"].shape[1], c["pos"], c["seq"], c["table_off"], c["tables"], c["k_pool"],
                            c["v_pool"], c["heads"], c["kv_heads"], c["D"], c["bs"])


# fp16 K/V/Q are exact on both sides; the kernel rounds P and the output to fp16 (2^-11
# relative each) and uses ex2.approx: 3e-3 of the row's largest output bounds their sum.
ATTN_TOL = 3e-3

DECODE_CASES = [
    # (D, heads, kv_heads, bs, contexts)
    (16, 4, 2, 16, [1, 15, 16, 17, 53, 511, 512, 513, 1300]),
    (32, 8, 8, 16, [1, 40, 1025]),
    (64, 32, 4, 16, [7, 600, 2048]),
    (128, 32, 8, 16, [1, 16, 100, 512, 513, 1024, 4096]),
    (128, 32, 8, 32, [33, 1000]),
    (128, 16, 1, 16, [3, 700]),       # 16 query heads on one KV head: the wide path
    (64, 12, 4, 1, [1, 9, 530]),      # block size 1: every key in its own block
    (64, 6, 2, 8, [5, 29, 1100]),     # block size below the 16-key tile
    (16, 4, 2, 48, [100, 777]),       # block size not a power of two
    (128, 8, 2, 16, [5000, 4097, 700, 3]),  # more than eight slices: partials in global memory and the merge kernel
    (64, 8, 8, 16, [6100, 1]),
    # one or two sequences: the grid fits the SMs, so the slices of a (token, KV head) run as one
    # cluster and merge on chip
    (128, 32, 8, 16, [4096]),         # 8 slices
    (128, 32, 8, 16, [3000]),         # 6 slices, the last one ragged
    (128, 32, 8, 16, [2048, 1500]),   # 4 slices; the shorter context leaves one of its own empty
    (128, 8, 2, 16, [4000]),
    (64, 16, 4, 16, [4096]),
]


@pytest.mark.parametrize("D,heads,kv_heads,bs,ctxs", DECODE_CASES)
def test_decode_attention_matches_oracle(ops, D, heads, kv_heads, bs, ctxs):
    nb = sum((c + bs - 1) // bs for c in ctxs) + 5
    case = paged_attention_case(10 + D, ctxs, [1] * len(ctxs), heads, kv_heads, D, bs, nb)
    got, want = run_attention(ops, case, "decode"), oracle_attention(case)
    assert row_err(got, want) < ATTN_TOL


def test_decode_attention_full_size_c2_shape(ops):
    # the benchmark's workload: 32 sequences, contexts uniform in [1024, 4096], 32 q / 8 kv heads, D 128
    ctxs = c2_contexts()
    case = paged_attention_case(2, ctxs, [1] * 32, 32, 8, 128, 16, 16384)
    got, want = run_attention(ops, case, "decode"), oracle_attention(case)
    assert row_err(got, want) < ATTN_TOL


@pytest.mark.parametrize("n_seqs,ctx,why", [
    (256, 4096, "2048 (token, KV head) pairs: one 4096-key slice per pair, written straight to the output, no merge"),
    (64, 4096, "512 pairs: one slice per pair as well, in fewer than two waves of CTAs"),
    (32, 9024, "256 pairs whose contexts exceed the 8192 keys a slice's table holds: two slices each, partials and the merge kernel"),
])
def test_decode_attention_at_the_decode_step_benchmark_size(ops, n_seqs, ctx, why):
    # The launch the headline decode step makes per layer: every sequence at one context, 32 q /
    # 8 kv heads of 128, block 16. With this many (token, KV head) pairs a slice is the whole
    # context (launch_decode_attention), a path the small cases above never take.
    heads, kv_heads, D, bs = 32, 8, 128, 16
    case = WideDecodeCase(5, n_seqs, ctx, heads, kv_heads, D, bs)
    k16, v16 = case.pools16()
    shape = ops.attn_shape(heads, kv_heads, D, bs)
    meta = ops.TokenMeta.from_host(case.pos, case.seq, case.table_off, case.tables)
    out = torch.zeros((n_seqs, heads * D), dtype=torch.float16, device="cuda")
    ops.decode_attention(shape, dev(case.q), meta, dev(np.arange(n_seqs, dtype=np.int32)), ctx, dev(k16), dev(v16), out)
    torch.cuda.synchronize()
    got = out.cpu().numpy().astype(np.float32)
    del k16, v16
    for g in range(n_seqs // case.group):  # the CPU checker, one group of sequences at a time
        want = oracle_attention(case.group_case(g))
        assert row_err(got[g * case.group:(g + 1) * case.group], want) < ATTN_TOL, (g, why)


PREFILL_CASES = [
    (16, 4, 2, 16, [37, 1, 64, 65, 200], [37, 1, 64, 65, 130]),   # whole prompts, a 1-row chunk, a late chunk
    (32, 8, 4, 16, [300, 129], [192, 129]),
    (64, 32, 4, 16, [512, 1024], [512, 512]),                     # the prefill workload's shape, chunks 1 and 2
    (128, 8, 2, 16, [700, 90], [300, 90]),
    (128, 32, 8, 16, [1100], [640]),                              # Llama-3-8B head layout
    (64, 8, 2, 32, [333, 64], [333, 1]),                          # block size 32: two 16-key pages per block
    (64, 4, 4, 1, [70], [70]),
    (64, 6, 2, 8, [150], [77]),
]


@pytest.mark.parametrize("D,heads,kv_heads,bs,ctxs,chunks", PREFILL_CASES)
def test_prefill_attention_matches_oracle(ops, D, heads, kv_heads, bs, ctxs, chunks):
    nb = sum((c + bs - 1) // bs for c in ctxs) + 3
    case = paged_attention_case(20 + D, ctxs, chunks, heads, kv_heads, D, bs, nb)
    got, want = run_attention(ops, case, "prefill"), oracle_attention(case)
    assert row_err(got, want) < ATTN_TOL


@pytest.mark.parametrize("D,heads,kv_heads,ctx,chunk", [(64, 8, 2, 1100, 640), (128, 8, 4, 900, 300), (64, 4, 2, 333, 333)])
def test_prefill_attention_with_peaked_scores_and_dirty_pool(ops, D, heads, kv_heads, ctx, chunk):
    # Scores three times wider than N(0,1) queries give: row maxima keep growing by several
    # octaves after the first key tile, so the running output is rescaled in later tiles too.
    # Cache slots past the context hold NaN: nothing outside the context may reach a result.
    bs = 16
    nb = (ctx + bs - 1) // bs + 2
    case = paged_attention_case(50 + D, [ctx], [chunk], heads, kv_heads, D, bs, nb)
    case["q"] = (case["q"] * 3).astype(np.float16).astype(np.float32)
    want = oracle_attention(case)
    dirty = dict(case)
    used = np.zeros((nb, bs), bool)
    for j in range(ctx):
        used[case["tables"][case["table_off"][0] + j // bs], j % bs] = True
    for name in ("k_pool", "v_pool"):
        pool = case[name].copy()  # [blocks, kv heads, slots, D]
        pool[np.broadcast_to(~used[:, None, :, None], pool.shape)] = np.nan
        dirty[name] = pool
    got = run_attention(ops, dirty, "prefill")
    assert np.isfinite(got).all()
    assert row_err(got, want) < ATTN_TOL


@pytest.mark.parametrize("D,heads,kv_heads,bs", [(8, 8, 2, 16), (16, 4, 2, 16), (128, 32, 8, 16), (96, 6, 3, 4), (256, 2, 1, 16)])
def test_reference_attention_matches_oracle(ops, D, heads, kv_heads, bs):
    ctxs, chunks = [1, 130, 300], [1, 60, 1]
    nb = sum((c + bs - 1) // bs for c in ctxs) + 3
    case = paged_attention_case(30 + D, ctxs, chunks, heads, kv_heads, D, bs, nb)
    got, want = run_attention(ops, case, "reference"), oracle_attention(case)
    assert row_err(got, want) < 1e-3  # fp32 P and accumulation; only the fp16 output rounds


def test_prefill_2048_tokens_in_four_chunks_equals_one_pass(ops):
    # the prefill workload: 32 q / 4 kv heads, D 64, four 512-token chunks over the growing cache
    D, heads, kv_heads, bs = 64, 32, 4, 16
    whole = paged_attention_case(7, [2048], [2048], heads, kv_heads, D, bs, 140)
    want = oracle_attention(whole)
    got_whole = run_attention(ops, whole, "prefill")
    assert row_err(got_whole, want) < ATTN_TOL
    for c in range(4):
        part = dict(whole)
        lo, hi = 512 * c, 512 * (c + 1)
        part["q"], part["pos"], part["seq"] = whole["q"][lo:hi], whole["pos"][lo:hi], whole["seq"][lo:hi]
        part["ctxs"], part["chunk_lens"] = [hi], [512]
        got = run_attention(ops, part, "prefill")
        assert np.array_equal(got, got_whole[lo:hi])  # same tiles, same keys: identical bits


# ---- linear layers ----------------------------------------------------------------------------

def linear_case(seed, T, K, N, int8):
    rng = np.random.Generator(np.random.PCG64(seed))
    x = round_f16(rng.standard_normal((T, K)))
    y0 = rng.standard_normal((T, N)).astype(np.float32)
    if int8:
        wq = rng.integers(-127, 128, (N, K)).astype(np.int8)
        scale = rng.uniform(0.001, 0.02, N).astype(np.float32)
        return x, y0, wq, scale
    w = round_f16(rng.standard_normal((N, K)) * 0.05)
    return x, y0, w, None


def linear_oracle(x, y0, w, scale, beta):
    if scale is not None:
        return oracle.gemv_int8(w, scale, x, y=y0 if beta else None, beta=beta)
    y = (x.astype(np.float64) @ w.astype(np.float64).T).astype(np.float32)
    return y + beta * y0 if beta else y


# Products of fp16-exact inputs summed in fp32 in a different order than the oracle's
# double: K * 2^-24 relative to sum|w x| in the worst case; 1e-4 of the row's largest output.
LINEAR_TOL = 1e-4

GEMV_SHAPES = [(64, 256), (192, 64), (4096, 4096), (4096, 1024), (4096, 14336), (14336, 4096), (4096, 1000), (128, 72), (4160, 1024)]


@pytest.mark.parametrize("K,N", GEMV_SHAPES)
@pytest.mark.parametrize("int8", [True, False])
def test_gemv_matches_oracle(ops, K, N, int8):
    for T, beta in [(1, 0.0), (2, 1.0), (4, 0.0), (8, 1.0), (5, 0.0)]:
        x, y0, w, scale = linear_case(K + N + T, T, K, N, int8)
        want = linear_oracle(x, y0, w, scale, beta)
        y = dev(y0)
        scratch = ops.gemv_scratch(N, K)
        for _ in range(2):  # twice on the same scratch: it must come back clean
            y.copy_(dev(y0))
            if int8:
                ops.gemv_int8(dev(w), dev(scale), dev(x, torch.float16), y, beta, scratch)
            else:
                ops.gemv_f16(dev(w, torch.float16), dev(x, torch.float16), y, beta, scratch)
            assert row_err(y.cpu().numpy(), want) < LINEAR_TOL


@pytest.mark.parametrize("K,N", [(64, 256), (192, 64), (4096, 4096), (4096, 1024), (14336, 4096), (4096, 14336), (4096, 1000)])
@pytest.mark.parametrize("int8", [True, False])
def test_gemm_matches_oracle(ops, K, N, int8):
    for T, beta in [(9, 0.0), (64, 1.0), (100, 0.0), (256, 1.0)]:
        if int8 and K * N * T > 4096 * 4096 * 64 and T > 64:
            continue  # keep the CPU restatement of the int8 product in seconds (fp16 is checked by a float64 matmul)
        x, y0, w, scale = linear_case(K + N + T, T, K, N, int8)
        want = linear_oracle(x, y0, w, scale, beta)
        y = dev(y0)
        ops.gemm(dev(w) if int8 else dev(w, torch.float16), dev(x, torch.float16), y, beta, dev(scale) if int8 else None)
        torch.cuda.synchronize()
        assert ops.gemm_status() == 0  # no pipeline wait of the tensor-core kernel gave up
        assert row_err(y.cpu().numpy(), want) < LINEAR_TOL


@pytest.mark.parametrize("T", [1, 4, 5, 16])
def test_int8_linear_with_outlier_zero_and_tiny_activation_rows(ops, T):
    # The int8 few-token kernel rewrites each activation row as fixed-point digits relative to
    # the row's largest magnitude (inside the GEMM up to 4 tokens, in a kernel of its own above): rows with one huge outlier, all-zero rows, rows of fp16
    # subnormals and rows at the fp16 maximum must all stay within the linear tolerance.
    K, N = 4096, 4096
    rng = np.random.Generator(np.random.PCG64(5 + T))
    x = round_f16(rng.standard_normal((T, K)))
    x[0] = 0.0
    if T > 1:
        x[1] = round_f16(rng.standard_normal(K) * 1e-3)
        x[1, 17] = -60000.0
        x[2] = round_f16(rng.standard_normal(K) * 3e-7)  # fp16 subnormals
        x[3] = np.where(rng.random(K) < 0.5, 65504.0, -65504.0) * (rng.random(K) < 0.01)
    if T > 4:
        x[4, :] = round_f16(rng.standard_normal(K))
        x[4, K - 1] = 2048.0
    wq = rng.integers(-127, 128, (N, K)).astype(np.int8)
    scale = rng.uniform(0.001, 0.02, N).astype(np.float32)
    want = oracle.gemv_int8(wq, scale, x)
    y = torch.zeros((T, N), device="cuda")
    if T in (1, 5):
        ops.gemv_int8(dev(wq), dev(scale), dev(x, torch.float16), y, 0.0, ops.gemv_scratch(N, K))
    else:  # no scratch: 4 tokens take the kernel that makes the digits itself
        ops.gemm(dev(wq), dev(x, torch.float16), y, 0.0, dev(scale))
    torch.cuda.synchronize()
    assert ops.gemm_status() == 0
    got = y.cpu().numpy()
    assert np.array_equal(got[0], np.zeros(N, np.float32))  # a zero row gives exact zeros
    assert np.isfinite(got).all()
    assert row_err(got[1:], want[1:]) < LINEAR_TOL if T > 1 else True


@pytest.mark.parametrize("K,N", [(4160, 1024), (4096, 4096), (14336, 4096), (4096, 14336)])
def test_int8_few_tokens_without_scratch_make_their_digits_in_the_kernel(ops, K, N):
    # Up to 4 tokens and no digit buffer: the CTAs find the row maxima and write the digit tiles
    # into the shared-memory ring themselves (K = 4160 ends in a half k block; 4096 -> 4096 and
    # 14336 -> 4096 split K over a cluster).
    for T, beta in [(1, 1.0), (3, 0.0), (4, 1.0)]:
        x, y0, wq, scale = linear_case(K + N + T + 7, T, K, N, True)
        want = linear_oracle(x, y0, wq, scale, beta)
        y = dev(y0)
        ops.gemm(dev(wq), dev(x, torch.float16), y, beta, dev(scale))
        torch.cuda.synchronize()
        assert ops.gemm_status() == 0
        assert row_err(y.cpu().numpy(), want) < LINEAR_TOL
        again = ops.gemm(dev(wq), dev(x, torch.float16), dev(y0), beta, dev(scale))
        assert torch.equal(again, y)


def test_gemv_and_gemm_agree_and_are_deterministic(ops):
    x, y0, w, scale = linear_case(99, 8, 4096, 4096, True)
    a = ops.gemv_int8(dev(w), dev(scale), dev(x, torch.float16), torch.zeros((8, 4096), device="cuda"))
    b = ops.gemv_int8(dev(w), dev(scale), dev(x, torch.float16), torch.zeros((8, 4096), device="cuda"))
    assert torch.equal(a, b)  # split-K partials are added in a fixed order
    c = ops.gemm(dev(w), dev(x, torch.float16), torch.zeros((8, 4096), device="cuda"), 0.0, dev(scale))
    assert row_err(c.cpu().numpy(), a.cpu().numpy()) < LINEAR_TOL


def test_linear_rejects_bad_shapes(ops):
    w = torch.zeros((64, 100), dtype=torch.int8, device="cuda")
    with pytest.raises(ValueError, match="multiple of 64"):
        ops.gemv_int8(w, torch.ones(64, device="cuda"), torch.zeros((1, 100), dtype=torch.float16, device="cuda"),
                      torch.zeros((1, 64), device="cuda"))
    w = torch.zeros((64, 128), dtype=torch.int8, device="cuda")
    with pytest.raises(ValueError, match="at most 8"):
        ops.gemv_int8(w, torch.ones(64, device="cuda"), torch.zeros((9, 128), dtype=torch.float16, device="cuda"),
                      torch.zeros((9, 64), device="cuda"))


@pytest.mark.parametrize("splits", [2, 4, 8])
def test_linear_layers_with_a_forced_cluster_k_split(splits):
    # RB200_GEMM_SPLITS is read once per process, so each split factor gets a process of its own:
    # the tcgen05 GEMMs (fp16, int8 widening, int8 few-token) then split K over a cluster of that
    # size on every shape that allows it, and must still match the CPU checker.
    import os
    import subprocess
    import sys
    env = dict(os.environ, RB200_GEMM_SPLITS=str(splits))
    sel = "(test_gemm_matches_oracle or test_gemv_matches_oracle or test_int8_few_tokens) and (4096-4096 or 14336-4096 or 4160-1024)"
    r = subprocess.run([sys.executable, "-m", "pytest", "-x", "-q", "-m", "gpu", os.path.abspath(__file__), "-k", sel,
                        "-p", "no:cacheprovider"], env=env, capture_output=True, text=True, timeout=1200,
                       cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
    assert " passed" in r.stdout and "no tests ran" not in r.stdout
