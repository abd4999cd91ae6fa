"""The sampler on the device and the decode session (the step-with-deltas form of forward).

Sampler: the token and log-probability the device picks from a row of logits must be the ones
relay's host sampler picks from the same row (engine/src/sampler.cpp, called per row by
engine/src/engine.cpp:270-282): tokens identical, log-probabilities within 1e-6 (both sides
sum in float64; the order of the additions differs).

Session: a 64-step decode schedule with block growth, driven from device-resident state and
replayed as a CUDA graph, must give bit-identical logits and the same tokens as rb200_forward
fed the whole batch from the host on every step.
"""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from oracle import oracle  # noqa: E402  (the checker: tests only)
from relay_b200.types import ForwardBatch, SeqChunk  # noqa: E402
from tests.workloads import c1_inputs  # noqa: E402

LOGPROB_TOL = 1e-6


@pytest.fixture(scope="module")
def gpu():
    if not torch.cuda.is_available():
        pytest.fail("the gpu tests need a CUDA device")
    from relay_b200 import _lib, ops
    from relay_b200.backend import make_cuda_backend
    return _lib, ops, make_cuda_backend


def params_tensor(_lib, rows):
    """A device buffer of rb200_sampling_params from (temperature, top_p, top_k, seed, index) rows."""
    arr = (_lib.CSamplingParams * len(rows))()
    for i, (t, top_p, top_k, seed, index) in enumerate(rows):
        arr[i] = _lib.CSamplingParams(float(t), float(top_p), int(top_k), 0, int(seed), int(index))
    raw = np.frombuffer(bytes(arr), dtype=np.uint8).copy()
    return torch.from_numpy(raw).cuda()


def run_sampler(_lib, ops, logits, rows, logprobs=True):
    R = logits.shape[0]
    tok = torch.full((R,), -1, dtype=torch.int32, device="cuda")
    lp = torch.zeros(R, dtype=torch.float64, device="cuda") if logprobs else None
    ops.sample_rows(torch.from_numpy(logits).cuda(), params_tensor(_lib, rows), tok, lp)
    torch.cuda.synchronize()
    return tok.cpu().numpy(), (lp.cpu().numpy() if logprobs else None)


@pytest.mark.parametrize("V,R,spread", [(128256, 12, 3.0), (128256, 4, 12.0), (1000, 16, 2.0), (5, 8, 1.0), (4097, 6, 6.0)])
def test_sample_rows_picks_what_relays_sampler_picks(gpu, V, R, spread):
    _lib, ops, _ = gpu
    rng = np.random.Generator(np.random.PCG64(V + R))
    logits = (rng.standard_normal((R, V)) * spread).astype(np.float32)
    logits[0, [min(3, V - 1), V // 2, V - 1]] = logits[0].max() + 1.0  # a tie for the maximum: the lowest id wins
    rows = []
    for r in range(R):
        t = [0.0, 1.0, 0.7, 1.5, 0.05][r % 5]  # 0.05: nearly every term underflows to zero
        rows.append((t, 1.0, 0 if r % 2 else V + 5, int(rng.integers(0, 2 ** 62)), int(rng.integers(0, 4096))))
    tok, lp = run_sampler(_lib, ops, logits, rows)
    for r in range(R):
        want_tok, want_lp = oracle.sample(logits[r], *rows[r])
        assert tok[r] == want_tok, (r, rows[r])
        assert abs(lp[r] - want_lp) <= LOGPROB_TOL * max(1.0, abs(want_lp)), (r, rows[r])
    # without log-probabilities the same tokens come back
    tok2, _ = run_sampler(_lib, ops, logits, rows, logprobs=False)
    assert np.array_equal(tok, tok2)


TRUNCATED_CASES = [
    # (V, spread of the logits, [(temperature, top_p, top_k)])
    (128256, 3.0, [(0.8, 1.0, 50), (1.0, 0.9, 0), (0.7, 0.95, 1000), (1.3, 1.0, 1), (1.0, 0.5, 40), (1.0, 1.0, 5000),
                   (2.0, 0.999, 0), (1.0, 0.3, 2048), (0.9, 0.99, 2049)]),
    (128256, 0.02, [(1.0, 0.2, 0), (1.0, 1.0, 7000), (1.0, 0.05, 9000)]),  # nearly flat: nuclei of many thousand tokens
    (3000, 2.0, [(0.8, 0.9, 0), (1.0, 1.0, 10), (1.5, 0.7, 2999), (1.0, 0.999999, 0)]),
    (37, 1.0, [(1.0, 0.5, 3), (0.7, 0.9, 36), (1.0, 0.1, 0)]),
]


@pytest.mark.parametrize("V,spread,settings", TRUNCATED_CASES)
def test_truncated_sampling_picks_what_relays_sampler_picks(gpu, V, spread, settings):
    _lib, ops, _ = gpu
    rng = np.random.Generator(np.random.PCG64(V + len(settings)))
    R = 2 * len(settings)
    logits = (rng.standard_normal((R, V)) * spread).astype(np.float32)
    # equal logits at the top and in the body: candidates are then ordered by id
    logits[0, [V // 3, 2, V - 1]] = logits[0].max()
    logits[1] = np.round(logits[1] * 2) / 2
    rows = [settings[r % len(settings)] + (int(rng.integers(0, 2 ** 62)), int(rng.integers(0, 4096))) for r in range(R)]
    tok, lp = run_sampler(_lib, ops, logits, rows)
    for r in range(R):
        want_tok, want_lp = oracle.sample(logits[r], *rows[r])
        assert tok[r] == want_tok, (r, rows[r])
        assert abs(lp[r] - want_lp) <= LOGPROB_TOL * max(1.0, abs(want_lp)), (r, rows[r])


def test_sampled_tokens_follow_the_distribution_and_depend_only_on_seed_and_index(gpu):
    _lib, ops, _ = gpu
    V = 50
    rng = np.random.Generator(np.random.PCG64(8))
    row = (rng.standard_normal(V) * 1.5).astype(np.float32)
    n = 4000
    logits = np.tile(row, (n, 1))
    rows = [(1.0, 1.0, 0, 1234, i) for i in range(n)]
    tok, _ = run_sampler(_lib, ops, logits, rows, logprobs=False)
    assert [int(t) for t in tok[:200]] == [oracle.sample(row, *rows[i])[0] for i in range(200)]
    p = np.exp(row.astype(np.float64) - row.max())
    p /= p.sum()
    freq = np.bincount(tok, minlength=V) / n
    assert np.abs(freq - p).max() < 0.03
    # the same (seed, index) in another batch position gives the same token
    again, _ = run_sampler(_lib, ops, logits[:7], [rows[i] for i in (5, 4, 3, 2, 1, 0, 5)], logprobs=False)
    assert again.tolist() == [int(tok[i]) for i in (5, 4, 3, 2, 1, 0, 5)]


def test_forward_sample_equals_host_sampling_of_the_forward_logits(gpu):
    _lib, _, mk = gpu
    w, prompt, table = c1_inputs()
    be = mk(w, 64, 16)
    batch = ForwardBatch([SeqChunk(prompt.tolist(), 0, table.tolist())], all_logits=True)
    logits = be.forward(batch)
    rows = [([0.0, 0.8, 1.0, 1.3][i % 4], 1.0, 0, 99 + i, i) for i in range(len(prompt))]
    tok, lp = be.forward_sample(batch, rows, logprobs=True)
    for i, row in enumerate(rows):
        want_tok, want_lp = oracle.sample(logits[i], *row)
        assert tok[i] == want_tok
        assert abs(lp[i] - want_lp) <= LOGPROB_TOL * max(1.0, abs(want_lp))
    assert np.array_equal(be.forward_sample(batch, rows), tok)
    # greedy rows agree with the greedy entry point
    g_tok, _ = be.forward_greedy(batch)
    assert np.array_equal(be.forward_sample(batch, [(0.0, 1.0, 0, 0, 0)] * len(prompt)), g_tok)
    # rows with top-k / nucleus truncation mixed among the others
    mixed = [(0.9, [1.0, 0.9, 0.5][i % 3], [0, 5, 40, 300][i % 4], 7 + i, i) for i in range(len(prompt))]
    tok, lp = be.forward_sample(batch, mixed, logprobs=True)
    for i, row in enumerate(mixed):
        want_tok, want_lp = oracle.sample(logits[i], *row)
        assert tok[i] == want_tok, (i, row)
        assert abs(lp[i] - want_lp) <= LOGPROB_TOL * max(1.0, abs(want_lp))


# ---- decode sessions ---------------------------------------------------------------------------

def prefill_all(be, prompts, tables):
    last = []
    for p, t in zip(prompts, tables):
        lg = be.forward(ForwardBatch([SeqChunk(p, 0, t)]))
        last.append(int(np.argmax(lg[0])))
    return last


def session_case(cfg_vocab, bs, steps, seed=3):
    """Five sequences whose prompt lengths sit just before, on and after block boundaries, with the
    blocks each will need over `steps` steps drawn from a shuffled pool."""
    rng = np.random.Generator(np.random.PCG64(seed))
    lens = [bs - 1, bs, 2 * bs + 3, 5, 3 * bs - 2]
    prompts = [rng.integers(0, cfg_vocab, n).tolist() for n in lens]
    need = [(n + steps + bs) // bs + 1 for n in lens]
    pool = rng.permutation(sum(need) + 4).tolist()
    blocks, at = [], 0
    for k in need:
        blocks.append(pool[at:at + k])
        at += k
    return lens, prompts, blocks, at + 4


@pytest.mark.parametrize("model", ["c1", "d128_g4"])
def test_session_steps_equal_forward_bit_for_bit_over_64_steps_with_block_growth(gpu, model):
    _lib, _, mk = gpu
    from tests.test_gpu_model import WIDE_CONFIGS, synthetic
    if model == "c1":
        w, _, _ = c1_inputs()
    else:
        w = synthetic(WIDE_CONFIGS[model], 12)
    cfg, bs, steps = w.config, 16, 64
    lens, prompts, blocks, nblk = session_case(cfg.vocab, bs, steps)
    a, b = mk(w, nblk, bs), mk(w, nblk, bs)
    # both backends prefill with the blocks each prompt needs
    have = [(n + bs - 1) // bs for n in lens]
    first_a = prefill_all(a, prompts, [blk[:h] for blk, h in zip(blocks, have)])
    first_b = prefill_all(b, prompts, [blk[:h] for blk, h in zip(blocks, have)])
    assert first_a == first_b
    b.decode_open(lens, [blk[:h] for blk, h in zip(blocks, have)])
    ctx, toks = list(lens), list(first_a)
    for step in range(steps):
        new = []
        for s in range(len(lens)):
            if ctx[s] // bs + 1 > have[s]:  # the position about to be written opens a new block
                new.append((s, blocks[s][have[s]]))
                have[s] += 1
        want = a.forward(ForwardBatch([SeqChunk([toks[s]], ctx[s], blocks[s][:have[s]]) for s in range(len(lens))]))
        # step 0 gives the first tokens from the host; later steps feed what the device picked
        got = b.decode_step(tokens=toks if step == 0 else None, new_blocks=new, want_logits=True)
        assert np.array_equal(got["logits"], want), step
        toks = [int(np.argmax(r)) for r in want]
        assert got["tokens"].tolist() == toks, step
        ctx = [c + 1 for c in ctx]
    # the pages both wrote are the same bytes
    for layer in range(cfg.layers):
        for s in range(len(lens)):
            assert np.array_equal(a.read_kv_layer(layer, blocks[s][:have[s]]), b.read_kv_layer(layer, blocks[s][:have[s]]))
    b.decode_close()


def test_session_refuses_a_step_without_the_block_it_needs_and_keeps_its_state(gpu):
    _lib, _, mk = gpu
    w, _, _ = c1_inputs()
    bs = 16
    be, ref = mk(w, 32, bs), mk(w, 32, bs)
    prompt = list(range(1, bs + 1))  # exactly one block: the next position needs a second one
    for x in (be, ref):
        x.forward(ForwardBatch([SeqChunk(prompt, 0, [7])]))
    be.decode_open([bs], [[7]])
    with pytest.raises(ValueError, match="block table too short"):
        be.decode_step(tokens=[5])
    with pytest.raises(IndexError, match="token id out of range"):
        be.decode_step(tokens=[w.config.vocab], new_blocks=[(0, 9)])
    with pytest.raises(ValueError, match="block id out of range"):
        be.decode_step(tokens=[5], new_blocks=[(0, 32)])
    with pytest.raises(ValueError, match="picked none"):
        be.decode_step(tokens=None, new_blocks=[(0, 9)])
    got = be.decode_step(tokens=[5], new_blocks=[(0, 9)], want_logits=True)
    want = ref.forward(ForwardBatch([SeqChunk([5], bs, [7, 9])]))
    assert np.array_equal(got["logits"], want)


def test_session_slot_replacement_and_sampling(gpu):
    _lib, _, mk = gpu
    w, _, _ = c1_inputs()
    bs = 16
    be, ref = mk(w, 48, bs), mk(w, 48, bs)
    rng = np.random.Generator(np.random.PCG64(4))
    prompts = [rng.integers(0, 256, n).tolist() for n in (9, 20, 30)]
    tables = [[1, 2, 3], [10, 11, 12], [20, 21, 22]]
    for x in (be, ref):
        for p, t in zip(prompts, tables):
            x.forward(ForwardBatch([SeqChunk(p, 0, t)]))
    be.decode_open([9, 20], tables[:2])
    toks, ctx, seqs = [3, 4], [9, 20], [0, 1]
    for step in range(6):
        if step == 3:  # sequence 1 finishes; its slot goes to sequence 2
            be.decode_set_slot(1, 30, tables[2])
            seqs, ctx[1], toks[1] = [0, 2], 30, 8
        sampling = [(0.9, 1.0, 0, 1000 + seqs[s], step) for s in range(2)]
        batch = ForwardBatch([SeqChunk([toks[s]], ctx[s], tables[seqs[s]]) for s in range(2)])
        want_tok, want_lp = ref.forward_sample(batch, sampling, logprobs=True)
        feed = None if step not in (0, 3) else toks  # after a slot change the host names the tokens again
        got = be.decode_step(tokens=feed, sampling=sampling, logprobs=True)
        assert got["tokens"].tolist() == want_tok.tolist(), step
        assert np.array_equal(got["logprobs"], want_lp), step
        toks, ctx = want_tok.tolist(), [c + 1 for c in ctx]
