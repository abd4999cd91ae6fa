"""The whole forward pass on the GPU, through the host-side mirror of relay::Backend and the
C boundary, against the CPU oracle and the committed golden vectors.

Bars (the path's stated ones): logits within 2e-3 by the reference's own metric
(max|a-b| / max|b| per row, tests/test_reference.cpp:50-57) with identical greedy argmax;
KV pages and block-table moves bit-exact.
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from oracle import oracle  # noqa: E402
from relay_b200.types import CudaOptions, ForwardBatch, HostWeights, ModelConfig, SeqChunk  # noqa: E402
from tests.helpers import FIXTURES, GOLDEN, argmax_lowest, load_fixture, rel_err_rows  # noqa: E402
from tests.workloads import c1_inputs, round_f16  # noqa: E402

LOGIT_TOL = 2e-3


@pytest.fixture(scope="module")
def mk():
    if not torch.cuda.is_available():
        pytest.fail("the gpu tests need a CUDA device")
    from relay_b200.backend import make_cuda_backend
    return make_cuda_backend


def test_c1_tiny_llama_matches_cpu_reference_logits_and_greedy_tokens(mk):
    z = np.load(f"{GOLDEN}/c1_cpu_reference.npz")
    w, prompt, table = c1_inputs()
    be = mk(w, 64, 16)
    assert be.name() == "b200"
    lg = be.forward(ForwardBatch([SeqChunk(prompt.tolist(), 0, table.tolist())], all_logits=True))
    assert lg.shape == z["prompt_logits"].shape
    assert rel_err_rows(lg, z["prompt_logits"]) < LOGIT_TOL
    tok = argmax_lowest(lg[-1])
    for s in range(16):
        assert tok == int(z["tokens"][s])
        row = be.forward(ForwardBatch([SeqChunk([tok], 37 + s, table.tolist())]))[0]
        assert rel_err_rows(row[None], z["step_logits"][s][None]) < LOGIT_TOL
        tok = argmax_lowest(row)
    # the page the CPU backend wrote, rounded to the cache's fp16: equal up to one fp16 step
    k, v = be.read_kv_block(1, int(table[0]))
    for got, want in ((k, z["layer1_block0_k"]), (v, z["layer1_block0_v"])):
        g = got.view(np.float16).astype(np.float32)
        assert np.abs(g - want).max() <= 2e-3 * np.abs(want).max()


@pytest.mark.parametrize("name", FIXTURES)
def test_fixtures_match_transformers_golden_logits(mk, name):
    # tests/test_reference.cpp:77-119 of the reference, at this path's 2e-3 instead of its 2e-2
    w, gold = load_fixture(name)
    be = mk(w, 64, 16)
    prompt, table = gold["prompt"].tolist(), list(range(8))
    lg = be.forward(ForwardBatch([SeqChunk(prompt, 0, table)], all_logits=True))
    assert rel_err_rows(lg, gold["prompt_logits"]) < LOGIT_TOL
    tok, toks = argmax_lowest(lg[-1]), []
    for s in range(len(gold["generated"])):
        toks.append(tok)
        row = be.forward(ForwardBatch([SeqChunk([tok], len(prompt) + s, table)]))[0]
        if s + 1 < len(gold["step_logits"]):
            assert rel_err_rows(row[None], gold["step_logits"][s + 1][None]) < LOGIT_TOL
        tok = argmax_lowest(row)
    assert toks == gold["generated"].tolist()


def synthetic(cfg: ModelConfig, seed: int, std=0.05):
    return HostWeights.random(cfg, seed, std=std, norm_std=0.1)


WIDE_CONFIGS = {
    # head sizes the reference's fixtures do not reach (D = 64 and 128), still CPU-checkable
    "d128_g4": ModelConfig(hidden=256, intermediate=320, layers=2, heads=4, kv_heads=1, head_dim=128, vocab=512),
    "d64_g8": ModelConfig(hidden=256, intermediate=172, layers=2, heads=8, kv_heads=1, head_dim=64, vocab=300,
                          rope_theta=500000.0, rope_scaling_type="llama3", rope_factor=8.0,
                          rope_original_max_position=64.0),
    "d32_mha_bias": ModelConfig(hidden=128, intermediate=200, layers=3, heads=4, kv_heads=4, head_dim=32, vocab=260,
                                qkv_bias=True, tie_embeddings=True),
}


def schedule(cfg, rng, lens, chunk, steps, bs, first_block=0):
    """Chunked prefill of several sequences per pass, then decode steps with a fresh prompt
    riding along on odd steps (the shape of tests/test_attention.cpp:43-138)."""
    seqs, nxt = [], first_block
    extra = (40 + steps + bs - 1) // bs
    for n in lens:
        need = (n + steps + 1 + bs - 1) // bs
        seqs.append(dict(tok=rng.integers(0, cfg.vocab, n + steps + 1).tolist(), n=n, table=list(range(nxt, nxt + need)), done=0))
        nxt += need
    passes = []
    while any(s["done"] < s["n"] for s in seqs):
        b = ForwardBatch()
        for s in seqs:
            k = min(s["n"] - s["done"], chunk)
            if k > 0:
                b.seqs.append(SeqChunk(s["tok"][s["done"]:s["done"] + k], s["done"], s["table"]))
                s["done"] += k
        passes.append(b)
    for d in range(steps):
        b = ForwardBatch()
        for s in seqs:
            b.seqs.append(SeqChunk([s["tok"][s["done"]]], s["done"], s["table"]))
            s["done"] += 1
        if d % 2 == 1:  # a throwaway prompt in blocks of its own
            b.seqs.append(SeqChunk(rng.integers(0, cfg.vocab, 40 + d).tolist(), 0, list(range(nxt, nxt + extra))))
        passes.append(b)
    return passes, nxt + extra


@pytest.mark.parametrize("name", list(WIDE_CONFIGS))
@pytest.mark.parametrize("bs", [16, 4])
def test_mixed_prefill_and_decode_schedule_matches_cpu(mk, name, bs):
    cfg = WIDE_CONFIGS[name]
    w = synthetic(cfg, 5)
    rng = np.random.Generator(np.random.PCG64(7))
    passes, blocks = schedule(cfg, rng, [1, 17, 64, 200, 700], 192, 6, bs)
    cpu = oracle.cpu_model(w, blocks, bs)
    gpu = mk(w, blocks, bs, max_batch_tokens=2048)
    worst, agree, total = 0.0, 0, 0
    for b in passes:
        a, g = cpu.forward(b), gpu.forward(b)
        assert a.shape == g.shape
        worst = max(worst, rel_err_rows(g, a))
        agree += int((a.argmax(1) == g.argmax(1)).sum())
        total += a.shape[0]
    assert worst < LOGIT_TOL
    assert agree == total


def test_batched_equals_alone_and_chunked_equals_whole_on_gpu(mk):
    # the invariances of tests/test_batching.cpp:75-120; on the GPU a token's kernels depend on
    # the batch (GEMV for up to 8 tokens, GEMM above; decode or prefill attention), each with
    # its own fp16 rounding of P and of the activations, so logits agree to that rounding
    # (about 2^-11 per rounding point) rather than bit for bit
    w = synthetic(WIDE_CONFIGS["d64_g8"], 9)
    rng = np.random.Generator(np.random.PCG64(3))
    p1, p2 = rng.integers(0, 300, 90).tolist(), rng.integers(0, 300, 23).tolist()
    t1, t2 = [5, 9, 2, 11, 30, 8], [7, 1]
    alone = mk(w, 32, 16).forward(ForwardBatch([SeqChunk(p1, 0, t1)], all_logits=True))
    both = mk(w, 32, 16).forward(ForwardBatch([SeqChunk(p2, 0, t2), SeqChunk(p1, 0, t1)], all_logits=True))
    assert rel_err_rows(both[len(p2):], alone) < 1.5e-3
    be = mk(w, 32, 16)
    rows = [be.forward(ForwardBatch([SeqChunk(p1[i:i + 7], i, t1)], all_logits=True)) for i in range(0, 90, 7)]
    assert rel_err_rows(np.concatenate(rows), alone) < 1.5e-3
    assert np.array_equal(np.concatenate(rows).argmax(1), alone.argmax(1))


def test_kv_blocks_moved_to_another_backend_decode_identically(mk):
    # tests/test_kv_cache.cpp:67-102 of the reference: prefill on A, copy its blocks to B under
    # different block ids, decode on both: same tokens; here also the same bits
    w, prompt, _ = c1_inputs()
    a, b = mk(w, 32, 16), mk(w, 32, 16)
    ta, tb = [3, 17, 9], [20, 1, 30]
    la = a.forward(ForwardBatch([SeqChunk(prompt.tolist(), 0, ta)]))
    for layer in range(w.config.layers):
        payload = a.read_kv_layer(layer, ta)
        b.write_kv_layer(layer, tb, payload)
        assert np.array_equal(b.read_kv_layer(layer, tb), payload)
        k, v = a.read_kv_block(layer, ta[1])
        k2, v2 = b.read_kv_block(layer, tb[1])
        assert np.array_equal(k, k2) and np.array_equal(v, v2)
    tok = argmax_lowest(la[0])
    for s in range(6):
        ra = a.forward(ForwardBatch([SeqChunk([tok], 37 + s, ta)]))[0]
        rb = b.forward(ForwardBatch([SeqChunk([tok], 37 + s, tb)]))[0]
        assert np.array_equal(ra, rb)
        tok = argmax_lowest(ra)


@pytest.mark.parametrize("layers_per_slot", [1, 2, 5])
def test_kv_link_moves_layer_ranges_between_two_backends(mk, layers_per_slot):
    # The prefill -> decode hop of a finished request over a K/V link joining two backends of this
    # process: whole layers per message, as many as a slot holds (a 5-layer model: 5, 3 and 1
    # messages); the received pages equal the sender's bit for bit, a dropped request moves the
    # ring on, and both backends decode the same tokens afterwards. Both ends share one GPU and one
    # host thread here, so the sender's work is always enqueued first and never has to wait for a
    # slot (8 slots, a host wait after every request): streams of one device may share a hardware
    # queue, and a wait enqueued ahead of the work that satisfies it could then block that work.
    # Slot reuse behind acknowledgements runs between processes in test_multi_gpu.py.
    cfg = ModelConfig(hidden=128, intermediate=200, layers=5, heads=4, kv_heads=2, head_dim=32, vocab=260)
    w = synthetic(cfg, 31)
    a, b = mk(w, 48, 16), mk(w, 48, 16)
    rng = np.random.Generator(np.random.PCG64(4))
    prompt = rng.integers(0, cfg.vocab, 150).tolist()
    ta, tb = list(range(2, 12)), list(range(30, 40))[::-1]
    la = a.forward(ForwardBatch([SeqChunk(prompt, 0, ta)]))
    slot = layers_per_slot * 2 * len(ta) * a.kv_block_bytes()
    (link_a, _), (link_b, _) = a.kv_link_create(8, slot), b.kv_link_create(8, slot)
    a.kv_link_connect_local(link_a, b, link_b)

    def settle():
        a.kv_link_wait(link_a, 20000)
        b.kv_link_wait(link_b, 20000)

    # a request the receiver drops, then the one it lands
    a.kv_link_send_layers(link_a, 0, cfg.layers, ta)
    settle()
    b.kv_link_skip_layers(link_b, cfg.layers, len(ta))
    settle()
    a.kv_link_send_layers(link_a, 0, cfg.layers, ta)
    settle()
    b.kv_link_recv_layers(link_b, 0, cfg.layers, tb)
    settle()
    for layer in range(cfg.layers):
        assert np.array_equal(b.read_kv_layer(layer, tb), a.read_kv_layer(layer, ta))
    # a range in the middle, into other blocks
    tc = list(range(12, 22))
    a.kv_link_send_layers(link_a, 1, 3, ta)
    settle()
    b.kv_link_recv_layers(link_b, 1, 3, tc)
    settle()
    for layer in (1, 2, 3):
        assert np.array_equal(b.read_kv_layer(layer, tc), a.read_kv_layer(layer, ta))
    tok = argmax_lowest(la[0])
    for s in range(4):
        ra = a.forward(ForwardBatch([SeqChunk([tok], 150 + s, ta)]))[0]
        rb = b.forward(ForwardBatch([SeqChunk([tok], 150 + s, tb)]))[0]
        assert np.array_equal(ra, rb)
        tok = argmax_lowest(ra)
    a.kv_link_close(link_a)
    b.kv_link_close(link_b)


def test_kv_pages_match_cpu_pages_rounded_to_fp16(mk):
    cfg = WIDE_CONFIGS["d128_g4"]
    w = synthetic(cfg, 2)
    rng = np.random.Generator(np.random.PCG64(1))
    toks = rng.integers(0, cfg.vocab, 50).tolist()
    table = [6, 2, 9, 0]
    cpu, gpu = oracle.cpu_model(w, 12, 16), mk(w, 12, 16)
    cpu.forward(ForwardBatch([SeqChunk(toks, 0, table)]))
    gpu.forward(ForwardBatch([SeqChunk(toks, 0, table)]))
    for layer in range(cfg.layers):
        for blk in table:
            kc, vc = cpu.read_kv_block(layer, blk)
            kg, vg = gpu.read_kv_block(layer, blk)
            for c, g in ((kc, kg), (vc, vg)):
                g = g.view(np.float16).astype(np.float32)
                assert np.abs(g - c).max() <= 2e-3 * np.abs(c).max()
    # slots past the 50 tokens stay zero, as on the CPU
    k, _ = gpu.read_kv_block(0, 0)
    assert np.all(k.view(np.float16).reshape(cfg.kv_heads, 16, cfg.head_dim)[:, 2:, :] == 0)


def test_layer_observer_fires_once_per_layer_in_order(mk):
    # tests/test_transfer.cpp:220-233
    w, prompt, table = c1_inputs()
    be = mk(w, 64, 16)
    seen = []
    be.forward(ForwardBatch([SeqChunk(prompt.tolist(), 0, table.tolist())]), observer=seen.append)
    assert seen == list(range(w.config.layers))
    for l in seen:
        be.wait_kv_written(l)


def test_forward_rejects_what_the_reference_rejects(mk):
    w, _, _ = c1_inputs()
    be = mk(w, 16, 16, max_batch_tokens=32, max_context=64)
    with pytest.raises(ValueError, match="block table too short"):
        be.forward(ForwardBatch([SeqChunk(list(range(17)), 0, [3])]))
    with pytest.raises(IndexError, match="token id out of range"):
        be.forward(ForwardBatch([SeqChunk([256], 0, [3])]))
    with pytest.raises(ValueError, match="max_context"):
        be.forward(ForwardBatch([SeqChunk([1], 64, [0, 1, 2, 3, 4])]))
    with pytest.raises(ValueError, match="max_batch_tokens"):
        be.forward(ForwardBatch([SeqChunk([1] * 33, 0, [0, 1, 2])]))
    with pytest.raises(ValueError, match="block id out of range"):
        be.forward(ForwardBatch([SeqChunk([1], 0, [16])]))
    assert be.forward(ForwardBatch([])).shape[0] == 0
    assert be.forward(ForwardBatch([SeqChunk([1, 2], 0, [1], want_logits=False)])).shape[0] == 0
    with pytest.raises(ValueError, match="no such layer"):
        be.read_kv_layer(99, [0])
    with pytest.raises(ValueError, match="wrong size"):
        be.update_weight("final_norm", np.zeros(3, np.float32))
    with pytest.raises(ValueError, match="no layers.9.wo"):
        be.update_weight("layers.9.wo", np.zeros(3, np.float32))


def test_reference_attention_option_agrees_with_the_fast_kernels(mk):
    # tests/test_attention.cpp:179-198 (M1 against M0): same logits up to rounding
    cfg = WIDE_CONFIGS["d64_g8"]
    w = synthetic(cfg, 4)
    rng = np.random.Generator(np.random.PCG64(5))
    passes, blocks = schedule(cfg, rng, [1, 17, 200, 700], 192, 4, 16)
    a = mk(w, blocks, 16, max_batch_tokens=2048, options=CudaOptions(reference_attention=True))
    b = mk(w, blocks, 16, max_batch_tokens=2048, options=CudaOptions())
    for p in passes:
        la, lb = a.forward(p), b.forward(p)
        assert rel_err_rows(lb, la) < LOGIT_TOL
        assert np.array_equal(la.argmax(1), lb.argmax(1))


def dequantised(w: HostWeights) -> HostWeights:
    """The float32 model an int8 backend represents: layer matrices replaced by q * scale."""
    out = dict(w.tensors)
    for name, t in w.tensors.items():
        if name.startswith("layers.") and t.ndim == 2:
            q, s = oracle.quantize_rows_int8(t)
            out[name] = (q.astype(np.float32) * s[:, None]).astype(np.float32)
    return HostWeights(w.config, out)


# Matrices on both sides of the size at which the int8 few-token linear changes kernels: QKV
# (1536 x 1024) and attention output (1024 x 1024) stay on the register GEMV, whose counters and
# partials live at the start of the backend's shared scratch; gate/up (5632 x 1024) and down
# (1024 x 2816) read int8 digits from the end of the same scratch.
MIXED_SIZE_CONFIG = ModelConfig(hidden=1024, intermediate=2816, layers=2, heads=8, kv_heads=2, head_dim=128, vocab=512)


@pytest.mark.parametrize("name", ["c1", "d128_g4", "mixed_sizes"])
def test_int8_weights_match_cpu_on_the_dequantised_model(mk, name):
    if name == "mixed_sizes":
        w = synthetic(MIXED_SIZE_CONFIG, 6, std=0.02)  # hidden 1024: the weight scale of the Llama-width model
    else:
        w = c1_inputs()[0] if name == "c1" else synthetic(WIDE_CONFIGS[name], 6)
    cfg = w.config
    rng = np.random.Generator(np.random.PCG64(8))
    passes, blocks = schedule(cfg, rng, [5, 60, 130], 64, 5, 16)
    cpu = oracle.cpu_model(dequantised(w), blocks, 16)
    gpu = mk(w, blocks, 16, max_batch_tokens=1024, options=CudaOptions(int8_weights=True))
    worst = 0.0
    for p in passes:
        a, g = cpu.forward(p), gpu.forward(p)
        worst = max(worst, rel_err_rows(g, a))
        assert np.array_equal(a.argmax(1), g.argmax(1))
    print(f"int8 {name}: rel err vs the dequantised model {worst:.2e}")
    assert worst < LOGIT_TOL


_WIDTH_MODEL = {}


def llama3_8b_width_model():
    if not _WIDTH_MODEL:  # 470 M weights take numpy a while: both variants share them
        cfg = ModelConfig(hidden=4096, intermediate=14336, layers=2, heads=32, kv_heads=8, head_dim=128, vocab=8192,
                          tie_embeddings=True, rope_theta=500000.0, rope_scaling_type="llama3", rope_factor=8.0,
                          rope_original_max_position=8192.0)
        _WIDTH_MODEL["w"] = HostWeights.random(cfg, 9, std=0.02, norm_std=0.1)
    return _WIDTH_MODEL["w"]


@pytest.mark.parametrize("int8", [False, True])
def test_llama3_8b_width_layers_match_cpu(mk, int8):
    # The widths of the decode benchmark's model (hidden 4096, 32 q / 8 kv heads of 128, SwiGLU
    # 14336, Llama-3 RoPE scaling), two layers and a reduced vocabulary so that relay's CPU backend
    # checks it in seconds: the projection shapes, head layout and context lengths the timed
    # kernels see (tcgen05 GEMMs with K = 4096 and 14336, the int8 digit kernel, tcgen05 prefill at
    # D = 128, split decode attention), under chunked prefill, 1- and 2-token decode steps.
    w = llama3_8b_width_model()
    cfg = w.config
    rng = np.random.Generator(np.random.PCG64(10))
    passes, blocks = schedule(cfg, rng, [300, 33], 256, 3, 16)
    # The model the device holds: int8 layer matrices times their scales, or every matrix rounded
    # to fp16 (as the reference's device upload does, engine/src/cuda_backend.cu:282-304). Against
    # that model the 2e-3 bar measures the compute path alone; against the unrounded float32
    # weights the storage rounding of 470 M weights adds to it.
    held = dequantised(w) if int8 else HostWeights(cfg, {n: (t if n.endswith("norm") else round_f16(t)) for n, t in w.tensors.items()})
    cpu_held, cpu_f32 = oracle.cpu_model(held, blocks, 16), oracle.cpu_model(w, blocks, 16)
    gpu = mk(w, blocks, 16, max_batch_tokens=512, options=CudaOptions(int8_weights=int8))
    worst_held, worst_f32 = 0.0, 0.0
    for p in passes:
        a, b, g = cpu_held.forward(p), cpu_f32.forward(p), gpu.forward(p)
        worst_held = max(worst_held, rel_err_rows(g, a))
        worst_f32 = max(worst_f32, rel_err_rows(g, b))
        assert np.array_equal(a.argmax(1), g.argmax(1))
        if not int8:
            assert np.array_equal(b.argmax(1), g.argmax(1))
    print(f"llama3-8b widths, int8={int8}: rel err vs the held model {worst_held:.2e}, vs float32 weights {worst_f32:.2e}")
    assert worst_held < LOGIT_TOL
    if not int8:
        assert worst_f32 < 1.5 * LOGIT_TOL


@pytest.mark.parametrize("lens", [[9, 5, 12, 7, 3, 10], [9, 5, 12, 7, 3, 10, 4, 6, 8, 2, 11]])
def test_llama3_8b_width_int8_few_sequence_steps_match_cpu(mk, lens):
    # 6- and 11-token decode steps: token counts at which every int8 projection reads its input as
    # int8 digits from a buffer — written by RMSNorm itself for the QKV and gate/up projections, by
    # the digit pass for the attention-output and down projections (up to 8 tokens through the
    # few-token entry of the linear layer, above through the general one).
    w = llama3_8b_width_model()
    cfg = w.config
    rng = np.random.Generator(np.random.PCG64(11))
    passes, blocks = schedule(cfg, rng, lens, 16, 3, 16)
    cpu = oracle.cpu_model(dequantised(w), blocks, 16)
    gpu = mk(w, blocks, 16, max_batch_tokens=128, options=CudaOptions(int8_weights=True))
    worst = 0.0
    for p in passes:
        a, g = cpu.forward(p), gpu.forward(p)
        worst = max(worst, rel_err_rows(g, a))
        assert np.array_equal(a.argmax(1), g.argmax(1))
    print(f"llama3-8b widths, int8, {len(lens)} sequences: rel err vs the held model {worst:.2e}")
    assert worst < LOGIT_TOL


def test_update_weight_equals_construction_and_accepts_device_pointers(mk):
    # tests/test_c_api.cpp (update_tensor == host write): a backend built empty and filled
    # tensor by tensor, half of them from device memory, gives the same bits
    w, prompt, table = c1_inputs()
    from relay_b200.backend import Backend
    batch = ForwardBatch([SeqChunk(prompt.tolist(), 0, table.tolist())], all_logits=True)
    for opts in (CudaOptions(), CudaOptions(int8_weights=True)):
        want = mk(w, 64, 16, options=opts).forward(batch)
        be = Backend(w.config, None, 64, 16, options=opts)
        keep = []
        for i, (name, t) in enumerate(w.tensors.items()):
            if i % 2:
                d = torch.from_numpy(t).cuda()
                keep.append(d)
                be.update_weight(name, d.data_ptr(), d.numel())
            else:
                be.update_weight(name, t)
        assert np.array_equal(be.forward(batch), want)


def test_forward_greedy_equals_host_argmax(mk):
    w, prompt, table = c1_inputs()
    be = mk(w, 64, 16, options=CudaOptions(gpu_argmax=True))
    b = ForwardBatch([SeqChunk(prompt.tolist(), 0, table.tolist())], all_logits=True)
    lg = be.forward(b)
    tok, val = be.forward_greedy(b)
    assert tok.tolist() == [argmax_lowest(r) for r in lg]
    assert np.array_equal(val, lg.max(1))


def test_concurrent_kv_reads_while_forward_runs(mk):
    # backend.h:60-64: read_kv_layer is safe from another thread during forward()
    import threading
    cfg = WIDE_CONFIGS["d64_g8"]
    w = synthetic(cfg, 3)
    be = mk(w, 64, 16, max_batch_tokens=1024)
    rng = np.random.Generator(np.random.PCG64(4))
    be.forward(ForwardBatch([SeqChunk(rng.integers(0, 300, 64).tolist(), 0, [0, 1, 2, 3])]))
    snap = [be.read_kv_layer(l, [0, 1, 2, 3]) for l in range(cfg.layers)]
    stop, bad = threading.Event(), []

    def reader():
        while not stop.is_set():
            for l in range(cfg.layers):
                if not np.array_equal(be.read_kv_layer(l, [0, 1, 2, 3]), snap[l]):
                    bad.append(l)

    th = threading.Thread(target=reader)
    th.start()
    for _ in range(20):  # forward passes on other blocks leave blocks 0-3 untouched
        be.forward(ForwardBatch([SeqChunk(rng.integers(0, 300, 500).tolist(), 0, list(range(8, 48)))]))
    stop.set()
    th.join()
    assert not bad
