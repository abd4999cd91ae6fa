"""Pins the CPU checkers (oracle/) before anything is compared against them.

The restatement is checked against (a) the reference's golden vectors — transformers logits
of its five fixtures, the tolerance of tests/test_reference.cpp:73 (1e-4) — (b) relay's own
CPU backend compiled from its sources, bit for bit, where oracle/_ref was built, (c) logits
that backend produced on the seeded tiny-Llama configuration (committed, so this holds
without the reference checkout), and (d) the reference's fp16 conversion known answers.
"""
import numpy as np
import pytest

from oracle import oracle
from relay_b200.types import ForwardBatch, HostWeights, ModelConfig, SeqChunk
from tests.helpers import FIXTURES, GOLDEN, argmax_lowest, load_fixture, rel_err_rows
from tests.workloads import c1_inputs

needs_ref = pytest.mark.skipif(not oracle.have_ref(), reason="relay's CPU backend was not compiled here (oracle/_ref)")


def test_f16_conversions_match_the_reference_known_answers():
    z = np.load(f"{GOLDEN}/f16_known_answers.npz")
    L = oracle.lib()
    got = np.asarray([L.ro_f16_to_f32(int(h)) for h in range(65536)], np.float32)
    assert np.array_equal(got.view(np.uint32), z["half_as_f32"].view(np.uint32))
    bits = oracle.f32_to_f16_bits(z["f32_in"])
    assert np.array_equal(bits, z["f16_bits"])
    # every half survives the round trip (tests/test_safetensors.cpp:32-39 of the reference)
    finite = ~np.isnan(z["half_as_f32"])
    back = oracle.f32_to_f16_bits(z["half_as_f32"][finite])
    assert np.array_equal(back, np.arange(65536, dtype=np.uint32).astype(np.uint16)[finite])
    # and agrees with IEEE round-to-nearest-even as numpy implements it
    with np.errstate(over="ignore"):
        assert np.array_equal(bits[~np.isnan(z["f32_in"])],
                              z["f32_in"][~np.isnan(z["f32_in"])].astype(np.float16).view(np.uint16))


@pytest.mark.parametrize("name", FIXTURES)
def test_restatement_matches_transformers_golden_logits(name):
    w, gold = load_fixture(name)
    m = oracle.OracleModel(w, 64, 16)
    prompt = gold["prompt"].tolist()
    table = list(range(8))
    lg = m.forward(ForwardBatch([SeqChunk(prompt, 0, table)], all_logits=True))
    assert lg.shape == gold["prompt_logits"].shape
    assert rel_err_rows(lg, gold["prompt_logits"]) < 1e-4
    toks, tok = [], argmax_lowest(lg[-1])
    for s in range(len(gold["generated"])):
        toks.append(tok)
        row = m.forward(ForwardBatch([SeqChunk([tok], len(prompt) + s, table)]))[0]
        tok = argmax_lowest(row)
        # step_logits[i] are the logits that chose generated[i]; [0] is the prompt's last row
        if s + 1 < len(gold["step_logits"]):
            assert rel_err_rows(row[None], gold["step_logits"][s + 1][None]) < 1e-4
    assert toks == gold["generated"].tolist()
    assert rel_err_rows(lg[-1:], gold["step_logits"][:1]) < 1e-4


def test_restatement_reproduces_committed_cpu_backend_logits_bit_for_bit():
    z = np.load(f"{GOLDEN}/c1_cpu_reference.npz")
    w, prompt, table = c1_inputs()
    assert np.array_equal(prompt, z["prompt"]) and np.array_equal(table, z["table"])
    m = oracle.OracleModel(w, 64, 16)
    lg = m.forward(ForwardBatch([SeqChunk(prompt.tolist(), 0, table.tolist())], all_logits=True))
    assert np.array_equal(lg, z["prompt_logits"])
    tok = argmax_lowest(lg[-1])
    for s in range(16):
        assert tok == int(z["tokens"][s])
        row = m.forward(ForwardBatch([SeqChunk([tok], 37 + s, table.tolist())]))[0]
        assert np.array_equal(row, z["step_logits"][s])
        tok = oracle.argmax(row)
    k, v = m.read_kv_block(1, int(table[0]))
    assert np.array_equal(k, z["layer1_block0_k"]) and np.array_equal(v, z["layer1_block0_v"])


def _random_schedule(cfg: ModelConfig, rng, n_seqs=3, bs=16, blocks=64):
    """A few prefill chunks and decode steps over shuffled block tables."""
    perm = rng.permutation(blocks).tolist()
    seqs = []
    for _ in range(n_seqs):
        n = int(rng.integers(1, 70))
        need = (n + 6 + bs - 1) // bs
        seqs.append({"tokens": rng.integers(0, cfg.vocab, n + 6).tolist(), "n": n, "table": [perm.pop() for _ in range(need)],
                     "done": 0})
    batches = []
    chunk = int(rng.integers(5, 40))
    while any(s["done"] < s["n"] for s in seqs):
        b = ForwardBatch()
        for s in seqs:
            left = s["n"] - s["done"]
            if left <= 0:
                continue
            k = min(left, chunk)
            b.seqs.append(SeqChunk(s["tokens"][s["done"]:s["done"] + k], s["done"], s["table"], True))
            s["done"] += k
        batches.append(b)
    for _ in range(5):
        b = ForwardBatch()
        for s in seqs:
            b.seqs.append(SeqChunk([s["tokens"][s["done"]]], s["done"], s["table"], True))
            s["done"] += 1
        batches.append(b)
    return batches


@needs_ref
@pytest.mark.parametrize("name", ["c1", "qwen2-bias", "llama3-rope", "llama-gqa-tied-bf16"])
def test_restatement_equals_relays_cpu_backend_bit_for_bit(name):
    w = c1_inputs()[0] if name == "c1" else load_fixture(name)[0]
    rng = np.random.Generator(np.random.PCG64(11))
    a, b = oracle.OracleModel(w, 64, 16), oracle.RefModel(w, 64, 16)
    for batch in _random_schedule(w.config, rng):
        la, lb = a.forward(batch), b.forward(batch)
        assert np.array_equal(la, lb)
    for layer in range(w.config.layers):
        for block in (0, 17, 63):
            ka, va = a.read_kv_block(layer, block)
            kb, vb = b.read_kv_block(layer, block)
            assert np.array_equal(ka, kb) and np.array_equal(va, vb)


@needs_ref
def test_helpers_equal_the_reference():
    R = oracle.ref_lib()
    for name in ("llama3-rope", "llama-mha"):
        cfg = load_fixture(name)[0].config
        mine = oracle.rope_inv_freq(cfg)
        theirs = np.zeros_like(mine)
        c = cfg.to_c()
        R.ref_rope_inv_freq(c, theirs.ctypes.data)
        assert np.array_equal(mine, theirs)
    row = np.asarray([1.0, 3.0, 3.0, -2.0, 3.0], np.float32)
    assert oracle.argmax(row) == R.ref_argmax(row.ctypes.data, row.size) == 1


def test_batched_equals_alone_and_chunked_equals_whole():
    # the bit-exact invariances tests/test_batching.cpp:75-120 of the reference relies on
    w = c1_inputs()[0]
    rng = np.random.Generator(np.random.PCG64(3))
    p1, p2 = rng.integers(0, 256, 45).tolist(), rng.integers(0, 256, 23).tolist()
    t1, t2 = [5, 9, 2], [7, 1]
    alone = oracle.OracleModel(w, 16, 16).forward(ForwardBatch([SeqChunk(p1, 0, t1)], all_logits=True))
    both = oracle.OracleModel(w, 16, 16).forward(ForwardBatch([SeqChunk(p2, 0, t2), SeqChunk(p1, 0, t1)], all_logits=True))
    assert np.array_equal(alone, both[len(p2):])
    m = oracle.OracleModel(w, 16, 16)
    rows = [m.forward(ForwardBatch([SeqChunk(p1[i:i + 7], i, t1)], all_logits=True)) for i in range(0, 45, 7)]
    assert np.array_equal(alone, np.concatenate(rows))


def test_forward_rejects_what_the_reference_rejects():
    w = c1_inputs()[0]
    m = oracle.OracleModel(w, 16, 16)
    with pytest.raises(ValueError, match="block table too short"):
        m.forward(ForwardBatch([SeqChunk(list(range(17)), 0, [3])]))
    with pytest.raises(ValueError, match="token id out of range"):
        m.forward(ForwardBatch([SeqChunk([256], 0, [3])]))
    assert m.forward(ForwardBatch([])).shape[0] == 0


def test_lse_merge_of_slices_equals_one_softmax():
    rng = np.random.Generator(np.random.PCG64(9))
    n, D, sl = 1300, 32, 512
    s = rng.standard_normal(n).astype(np.float32) * 3
    v = rng.standard_normal((n, D)).astype(np.float32)
    parts = (n + sl - 1) // sl + 1  # one empty slice at the end, as the reference launches
    po, pml = np.zeros((parts, D), np.float32), np.zeros((parts, 2), np.float32)
    for p in range(parts):
        sp, vp = s[p * sl:(p + 1) * sl], v[p * sl:(p + 1) * sl]
        if sp.size == 0:
            pml[p] = (-np.inf, 0)
            continue
        e = np.exp(sp - sp.max())
        pml[p] = (sp.max(), e.sum())
        po[p] = e @ vp
    e = np.exp(s - s.max())
    want = (e / e.sum()) @ v
    assert np.allclose(oracle.lse_merge(po, pml), want, rtol=1e-5, atol=1e-6)


def test_int8_quantisation_rule():
    w = np.asarray([[0.5, -1.27, 0.005, 0.015], [0, 0, 0, 0], [1e-3, 2.5e-3, -3.5e-3, 127e-3]], np.float32)
    q, s = oracle.quantize_rows_int8(w)
    assert np.allclose(s, [1.27 / 127, 1.0, 0.127 / 127])
    assert q[0].tolist() == [50, -127, 0, 2] or q[0].tolist() == [50, -127, 1, 2]  # 0.5 -> 0 under ties-to-even
    assert q[1].tolist() == [0, 0, 0, 0]
    assert q[2, 3] == 127
    x = np.ones((2, 4), np.float32)
    y = oracle.gemv_int8(q, s, x)
    assert np.allclose(y[0], (q.astype(np.float32) * s[:, None]).sum(1))
    y2 = oracle.gemv_int8(q, s, x, y=np.full((2, 3), 2.0, np.float32), beta=1.0)
    assert np.allclose(y2, y + 2.0)


def test_kv_gather_scatter_layout():
    rng = np.random.Generator(np.random.PCG64(2))
    bb, nb = 64, 10
    k = rng.integers(0, 255, nb * bb).astype(np.uint8)
    v = rng.integers(0, 255, nb * bb).astype(np.uint8)
    blocks = [7, 2, 9]
    st = oracle.kv_gather(k, v, blocks, bb)
    for i, b in enumerate(blocks):
        assert np.array_equal(st[i * bb:(i + 1) * bb], k[b * bb:(b + 1) * bb])
        assert np.array_equal(st[(3 + i) * bb:(4 + i) * bb], v[b * bb:(b + 1) * bb])
    k2, v2 = np.zeros_like(k), np.zeros_like(v)
    oracle.kv_scatter(k2, v2, [1, 0, 4], bb, st)
    assert np.array_equal(k2[bb:2 * bb], k[7 * bb:8 * bb]) and np.array_equal(v2[4 * bb:5 * bb], v[9 * bb:10 * bb])


def test_sampler_restatement_matches_the_reference_golden_rows():
    # tokens and log-probabilities relay's compiled sampler gave on these seeded rows (committed)
    from tests.workloads import sampler_cases
    z = np.load(f"{GOLDEN}/sampler_reference.npz")
    for i, (lg, t, top_p, top_k, seed, index) in enumerate(sampler_cases()):
        tok, lp = oracle.sample(lg, t, top_p, top_k, seed, index, prefer_reference=False)
        assert tok == int(z["tokens"][i]), (i, t, top_p, top_k)
        assert abs(lp - float(z["logprobs"][i])) <= 1e-12 * max(1.0, abs(lp))
    pairs = ((0, 0), (1, 0), (0, 1), (2 ** 63, 12345), (987654321, 2 ** 40))
    assert [oracle.uniform01(s, i) for s, i in pairs] == z["uniform01"].tolist()


@needs_ref
def test_sampler_restatement_equals_the_compiled_reference():
    from tests.workloads import sampler_cases
    for lg, t, top_p, top_k, seed, index in sampler_cases(seed=77, n=120):
        a = oracle.sample(lg, t, top_p, top_k, seed, index, prefer_reference=True)
        b = oracle.sample(lg, t, top_p, top_k, seed, index, prefer_reference=False)
        assert a[0] == b[0] and abs(a[1] - b[1]) <= 1e-12 * max(1.0, abs(a[1]))
