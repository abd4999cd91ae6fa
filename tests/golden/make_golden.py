"""Regenerates tests/golden/*.npz. Run where the reference checkout is present:

    python tests/golden/make_golden.py [/path/to/reference]

Two kinds of vectors, both produced by the reference itself (never by this repo's code):

* <fixture>.npz — the reference's five tiny-model fixtures (tests/fixtures/<name>/ of the
  reference): the float32 weights as relay's own loader fuses them (HostWeights::load,
  engine/src/weights.cpp:26-61, read back through oracle/ref_shim.cpp), the config, and the
  transformers logits of relay-reference.json (prompt logits at every position, 8 greedy
  tokens and their logits) that tests/test_reference.cpp:77-119 of the reference checks.
* c1_cpu_reference.npz — relay's float32 CPU backend (engine/src/cpu_backend.cpp, compiled
  unmodified into oracle/_ref) run on the seeded tiny Llama configuration: 37-token prompt,
  shuffled block table, 16 greedy steps; logits of every pass, the tokens, and one K/V page.
* f16_known_answers.npz — the reference's f32_to_f16 on the rounding cases of
  tests/test_safetensors.cpp:32-45 plus a seeded sample, and f16_to_f32 of all 65,536 halves.
"""
import dataclasses
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import oracle  # noqa: E402
from relay_b200.types import ForwardBatch, HostWeights, SeqChunk, tensor_shapes  # noqa: E402
from tests.workloads import c1_config, c1_inputs  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def fixture(ref_root: str, name: str) -> None:
    d = os.path.join(ref_root, "tests", "fixtures", name)
    m = oracle.RefModel(model_dir=d)
    cfg = m.config
    out = {"config_json": np.frombuffer(json.dumps(dataclasses.asdict(cfg)).encode(), dtype=np.uint8)}
    for tname, shape in tensor_shapes(cfg).items():
        t = m.tensor(tname)
        assert t is not None and t.size == int(np.prod(shape)), tname
        out["w:" + tname] = t.reshape(shape)
    with open(os.path.join(d, "relay-reference.json")) as f:
        ref = json.load(f)
    out["prompt"] = np.asarray(ref["prompt"], np.int32)
    out["generated"] = np.asarray(ref["generated"], np.int32)
    out["prompt_logits"] = np.asarray(ref["prompt_logits"], np.float32)
    out["step_logits"] = np.asarray(ref["step_logits"], np.float32)
    out["last_only"] = np.asarray(bool(ref.get("prompt_logits_last_only", False)))
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
    print(name, cfg, {k: v.shape for k, v in out.items() if not k.startswith("w:")})


def c1() -> None:
    cfg = c1_config()
    w, prompt, table = c1_inputs()
    m = oracle.RefModel(w, 64, 16)
    logits = [m.forward(ForwardBatch([SeqChunk(prompt.tolist(), 0, table.tolist())], all_logits=True))]
    toks = [int(np.argmax(logits[0][-1]))]
    step_logits = []
    for s in range(16):
        lg = m.forward(ForwardBatch([SeqChunk([toks[-1]], len(prompt) + s, table.tolist())]))
        step_logits.append(lg[0])
        toks.append(oracle.argmax(lg[0]))
    k0, v0 = m.read_kv_block(1, int(table[0]))
    np.savez_compressed(os.path.join(HERE, "c1_cpu_reference.npz"), prompt=prompt, table=table,
                        prompt_logits=logits[0], step_logits=np.stack(step_logits),
                        tokens=np.asarray(toks, np.int32), layer1_block0_k=k0, layer1_block0_v=v0)
    print("c1", cfg, "tokens", toks)


def f16() -> None:
    R = oracle.ref_lib()
    rng = np.random.Generator(np.random.PCG64(5))
    halves = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    as_f32 = np.asarray([R.ref_f16_to_f32(int(h)) for h in halves], np.float32)
    # rounding cases: exact halves, midpoints (ties), just above/below midpoints, subnormal
    # range, overflow threshold, infinities, NaN; then a seeded spread of magnitudes.
    cases = [0.0, -0.0, 1.0, -1.0, 65504.0, 65519.99, 65520.0, 65536.0, 1e10, -1e10, np.inf, -np.inf, np.nan,
             2.0 ** -24, 2.0 ** -25, 2.0 ** -25 * 1.0000001, 2.0 ** -26, 2.0 ** -14, 2.0 ** -14 - 2.0 ** -25,
             1.0 + 2.0 ** -11, 1.0 + 2.0 ** -10 + 2.0 ** -11, 1.0 + 2.0 ** -11 + 2.0 ** -20, 1.0 + 2.0 ** -11 - 2.0 ** -20,
             2047.5, 2048.5, 2049.0, 2051.0, 0.1, 0.2, 0.3, 3.14159265, 1e-5, 6e-8, 3e-8]
    sample = np.concatenate([np.asarray(cases, np.float32),
                             (rng.standard_normal(4096) * np.exp(rng.uniform(-20, 12, 4096))).astype(np.float32)])
    bits = np.asarray([R.ref_f32_to_f16(float(x)) for x in sample], np.uint16)
    np.savez_compressed(os.path.join(HERE, "f16_known_answers.npz"), half_as_f32=as_f32, f32_in=sample, f16_bits=bits)
    print("f16", sample.size, "cases")


def sampler() -> None:
    """relay's sampler (engine/src/sampler.cpp, compiled) on the seeded rows of
    tests/workloads.sampler_cases: the token and log-probability of every row."""
    from tests.workloads import sampler_cases
    R = oracle.ref_lib()
    toks, lps = [], []
    for lg, t, top_p, top_k, seed, index in sampler_cases():
        tok, lp = oracle.sample(lg, t, top_p, top_k, seed, index, prefer_reference=True)
        toks.append(tok)
        lps.append(lp)
    u = [R.ref_uniform01(s, i) for s, i in ((0, 0), (1, 0), (0, 1), (2 ** 63, 12345), (987654321, 2 ** 40))]
    np.savez_compressed(os.path.join(HERE, "sampler_reference.npz"), tokens=np.asarray(toks, np.int32),
                        logprobs=np.asarray(lps, np.float64), uniform01=np.asarray(u, np.float64))
    print("sampler", len(toks), "rows")


if __name__ == "__main__":
    ref_root = sys.argv[1] if len(sys.argv) > 1 else oracle.reference_root()
    if not ref_root:
        sys.exit("usage: python tests/golden/make_golden.py <root of the relay checkout>")
    oracle.build()
    for name in ("llama-mha", "llama-gqa-tied-bf16", "llama3-rope", "qwen2-bias", "chat-tiny"):
        fixture(ref_root, name)
    c1()
    f16()
    sampler()
