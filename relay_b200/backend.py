"""Host-side mirror of `relay::Backend` (engine/include/relay/backend.h:43-81) over the C
boundary: same methods, same argument meaning, same error behaviour (the reference's
std::invalid_argument / std::out_of_range become ValueError / IndexError).

    be = make_cuda_backend(weights, num_blocks, block_size, device, max_batch_tokens, max_context)
    logits = be.forward(ForwardBatch([SeqChunk(tokens, start_pos, block_table)]))
"""
from __future__ import annotations

import ctypes as C
from typing import Callable, List, Optional, Sequence, Tuple

import numpy as np

from . import _lib
from .types import (CModelConfig, CudaOptions, FlatBatch, ForwardBatch, HostWeights, ModelConfig, flatten, i32, ptr)


class KVLayout:
    """relay::KVLayout (engine/include/relay/kv_cache.h:22-36)."""

    def __init__(self, layers, kv_heads, head_dim, block_size, num_blocks):
        self.layers, self.kv_heads, self.head_dim = layers, kv_heads, head_dim
        self.block_size, self.num_blocks = block_size, num_blocks

    def block_elems(self) -> int:
        return self.kv_heads * self.block_size * self.head_dim

    def offset(self, block: int, kv_head: int, slot: int) -> int:
        return (block * self.kv_heads + kv_head) * self.block_size * self.head_dim + slot * self.head_dim

    def blocks_for(self, tokens: int) -> int:
        return (tokens + self.block_size - 1) // self.block_size


class Backend:
    def __init__(self, config: ModelConfig, weights: Optional[HostWeights], num_blocks: int, block_size: int,
                 device: int = 0, max_batch_tokens: int = 1024, max_context: Optional[int] = None,
                 options: Optional[CudaOptions] = None):
        self._L = _lib.lib()
        self._h = None
        options = CudaOptions.from_env() if options is None else options
        max_context = num_blocks * block_size if max_context is None else max_context
        cc = config.to_c()
        if weights is not None:
            cw, keep = weights.to_c()
            h = self._L.rb200_create(C.byref(cc), C.byref(cw), num_blocks, block_size, device, max_batch_tokens,
                                     max_context, options.flags())
            del keep
        else:
            h = self._L.rb200_create(C.byref(cc), None, num_blocks, block_size, device, max_batch_tokens, max_context,
                                     options.flags())
        if not h:
            _lib.raise_last_error()
        self._h = h
        self._config = config
        self._layout = KVLayout(config.layers, config.kv_heads, config.head_dim, block_size, num_blocks)
        self.options = options

    def close(self) -> None:
        if self._h:
            self._L.rb200_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- relay::Backend ---------------------------------------------------------------------
    def config(self) -> ModelConfig:
        return self._config

    def kv_layout(self) -> KVLayout:
        return self._layout

    def name(self) -> str:
        return self._L.rb200_name(self._h).decode()

    def _cb(self, observer):
        """The C callback for `observer`. An exception raised inside it cannot cross the C frames
        of the forward pass: it is kept (the first one) and re-raised by _reraise() once the
        call has returned."""
        self._cb_error = None
        if observer is None:
            return _lib.LAYER_CB(), None
        fn = observer.kv_written if hasattr(observer, "kv_written") else observer

        def call(_ctx, layer):
            if self._cb_error is None:
                try:
                    fn(layer)
                except BaseException as e:  # noqa: BLE001 - re-raised after the C call returns
                    self._cb_error = e

        cb = _lib.LAYER_CB(call)
        return cb, cb

    def _reraise(self):
        e, self._cb_error = getattr(self, "_cb_error", None), None
        if e is not None:
            raise e

    def forward_flat(self, fb: FlatBatch, observer=None, out: Optional[np.ndarray] = None) -> np.ndarray:
        """forward() on an already flattened batch; `out` may be a caller-owned (for example
        page-locked) float32 array of at least rows * vocab elements."""
        V = self._config.vocab
        rows = fb.n_rows
        if out is None:
            out = np.empty((max(rows, 1), V), np.float32)
        cb, keep = self._cb(observer)
        want = fb.want_logits.astype(np.uint8)
        r = self._L.rb200_forward(
            self._h, fb.n_seqs, ptr(fb.tokens), ptr(fb.chunk_len), ptr(fb.start_pos), ptr(fb.table_len), ptr(fb.tables),
            ptr(want), int(fb.all_logits), cb, None, out.ctypes.data_as(C.c_void_p), out.size)
        self._reraise()
        r = _lib.check(r)
        return out.reshape(-1)[: r * V].reshape(r, V)

    def forward(self, batch: ForwardBatch, observer=None) -> np.ndarray:
        """Backend::forward: [rows, vocab] float32, one row per chunk with want_logits (or per
        token with all_logits). `observer.kv_written(layer)` is called as each layer's K/V
        append is enqueued."""
        return self.forward_flat(flatten(batch), observer)

    def forward_greedy(self, batch: ForwardBatch, observer=None) -> Tuple[np.ndarray, np.ndarray]:
        """The greedy token and its logit per logits row, reduced on the device."""
        fb = flatten(batch)
        rows = max(fb.n_rows, 1)
        tok, val = np.empty(rows, np.int32), np.empty(rows, np.float32)
        cb, keep = self._cb(observer)
        want = fb.want_logits.astype(np.uint8)
        r = self._L.rb200_forward_greedy(
            self._h, fb.n_seqs, ptr(fb.tokens), ptr(fb.chunk_len), ptr(fb.start_pos), ptr(fb.table_len), ptr(fb.tables),
            ptr(want), int(fb.all_logits), cb, None, ptr(tok), ptr(val), rows)
        self._reraise()
        r = _lib.check(r)
        return tok[:r], val[:r]

    @staticmethod
    def _sampling_array(sampling, rows: int):
        """`sampling`: one (temperature, top_p, top_k, seed, index) tuple per logits row."""
        arr = (_lib.CSamplingParams * max(rows, 1))()
        if len(sampling) != rows:
            raise ValueError(f"sampling: {len(sampling)} entries for {rows} logits rows")
        for i, (t, top_p, top_k, seed, index) in enumerate(sampling):
            arr[i] = _lib.CSamplingParams(float(t), float(top_p), int(top_k), 0, int(seed), int(index))
        return arr

    def forward_sample(self, batch: ForwardBatch, sampling, logprobs: bool = False, observer=None):
        """The token relay's sampler picks from each logits row, sampled on the device, and (with
        `logprobs`) its log-probability. `sampling`: one (temperature, top_p, top_k, seed, index)
        per row."""
        fb = flatten(batch)
        rows = fb.n_rows
        arr = self._sampling_array(sampling, rows)
        tok = np.empty(max(rows, 1), np.int32)
        lp = np.empty(max(rows, 1), np.float64) if logprobs else None
        cb, keep = self._cb(observer)
        want = fb.want_logits.astype(np.uint8)
        r = self._L.rb200_forward_sample(
            self._h, fb.n_seqs, ptr(fb.tokens), ptr(fb.chunk_len), ptr(fb.start_pos), ptr(fb.table_len), ptr(fb.tables),
            ptr(want), int(fb.all_logits), cb, None, arr, ptr(tok), ptr(lp) if logprobs else None, rows)
        self._reraise()
        r = _lib.check(r)
        return (tok[:r], lp[:r]) if logprobs else tok[:r]

    # -- decode sessions (no counterpart in relay::Backend; see include/relay_b200.h) -------------
    def decode_open(self, context_lens: Sequence[int], tables: Sequence[Sequence[int]]) -> None:
        """A session over len(tables) sequences: slot s has context_lens[s] keys in the cache and the
        block ids tables[s] (spare ids allowed)."""
        ctx, tl = i32(context_lens), i32([len(t) for t in tables])
        flat = i32([b for t in tables for b in t]) if tl.sum() else i32([0])
        self._session_slots = len(tables)
        _lib.check(self._L.rb200_decode_open(self._h, len(tables), ptr(ctx), ptr(tl), ptr(flat)))

    def decode_set_slot(self, slot: int, context_len: int, table: Sequence[int]) -> None:
        t = i32(table) if len(table) else i32([0])
        _lib.check(self._L.rb200_decode_set_slot(self._h, slot, context_len, len(table), ptr(t)))

    def decode_step(self, tokens=None, new_blocks: Sequence[Tuple[int, int]] = (), sampling=None, want_tokens: bool = True,
                    logprobs: bool = False, want_logits: bool = False, logits_out: Optional[np.ndarray] = None):
        """One step of the open session. tokens: one id per slot, or None to feed the tokens the
        previous step picked on the device. new_blocks: (slot, block id) pairs appended since the
        last step. Returns a dict with the outputs asked for: "tokens", "logprobs", "logits"."""
        S, V = self._session_slots, self._config.vocab
        tok_in = i32(tokens) if tokens is not None else None
        if tok_in is not None and tok_in.size != S:
            raise ValueError("decode_step: one token per slot")
        nb_seq, nb_id = i32([s for s, _ in new_blocks]), i32([b for _, b in new_blocks])
        arr = self._sampling_array(sampling, S) if sampling is not None else None
        tok = np.empty(S, np.int32) if (want_tokens or sampling is not None or logprobs) else None
        lp = np.empty(S, np.float64) if logprobs else None
        lg = None
        if want_logits:
            lg = logits_out if logits_out is not None else np.empty((S, V), np.float32)
        _lib.check(self._L.rb200_decode_step(
            self._h, ptr(tok_in) if tok_in is not None else None, len(new_blocks), ptr(nb_seq) if len(new_blocks) else None,
            ptr(nb_id) if len(new_blocks) else None, arr, ptr(tok) if tok is not None else None,
            ptr(lp) if lp is not None else None, lg.ctypes.data_as(C.c_void_p) if lg is not None else None,
            lg.size if lg is not None else 0))
        out = {}
        if tok is not None:
            out["tokens"] = tok
        if lp is not None:
            out["logprobs"] = lp
        if lg is not None:
            out["logits"] = lg.reshape(-1)[: S * V].reshape(S, V)
        return out

    def decode_close(self) -> None:
        _lib.check(self._L.rb200_decode_close(self._h))

    def forward_greedy_flat(self, fb: FlatBatch) -> Tuple[np.ndarray, np.ndarray]:
        """forward_greedy() on an already flattened batch."""
        rows = max(fb.n_rows, 1)
        tok, val = np.empty(rows, np.int32), np.empty(rows, np.float32)
        want = fb.want_logits.astype(np.uint8)
        r = _lib.check(self._L.rb200_forward_greedy(
            self._h, fb.n_seqs, ptr(fb.tokens), ptr(fb.chunk_len), ptr(fb.start_pos), ptr(fb.table_len), ptr(fb.tables),
            ptr(want), int(fb.all_logits), _lib.LAYER_CB(), None, ptr(tok), ptr(val), rows))
        return tok[:r], val[:r]

    def kv_block_bytes(self) -> int:
        return self._L.rb200_kv_block_bytes(self._h)

    def read_kv_block(self, layer: int, block: int) -> Tuple[np.ndarray, np.ndarray]:
        bb = self.kv_block_bytes()
        k, v = np.empty(bb, np.uint8), np.empty(bb, np.uint8)
        _lib.check(self._L.rb200_read_kv_layer(self._h, layer, ptr(i32([block])), 1, ptr(k), ptr(v)))
        return k, v

    def write_kv_block(self, layer: int, block: int, k: np.ndarray, v: np.ndarray) -> None:
        k, v = np.ascontiguousarray(k).view(np.uint8), np.ascontiguousarray(v).view(np.uint8)
        if k.size != self.kv_block_bytes() or v.size != k.size:
            raise ValueError("write_kv_block: wrong block size")
        _lib.check(self._L.rb200_write_kv_layer(self._h, layer, ptr(i32([block])), 1, ptr(k), ptr(v)))

    def read_kv_layer(self, layer: int, blocks: Sequence[int]) -> np.ndarray:
        """All K blocks then all V blocks, in the order given (the transfer engine's payload)."""
        b = i32(blocks)
        bb = self.kv_block_bytes()
        out = np.empty(2 * b.size * bb, np.uint8)
        k = out.ctypes.data
        _lib.check(self._L.rb200_read_kv_layer(self._h, layer, ptr(b), b.size, C.c_void_p(k), C.c_void_p(k + b.size * bb)))
        return out

    def write_kv_layer(self, layer: int, blocks: Sequence[int], data: np.ndarray) -> None:
        b = i32(blocks)
        bb = self.kv_block_bytes()
        data = np.ascontiguousarray(data).view(np.uint8).ravel()
        if data.size != 2 * b.size * bb:
            raise ValueError("write_kv_layer: wrong payload size")
        k = data.ctypes.data
        _lib.check(self._L.rb200_write_kv_layer(self._h, layer, ptr(b), b.size, C.c_void_p(k), C.c_void_p(k + b.size * bb)))

    def kv_host_ptr(self, layer: int, block: int, value: bool):
        return None  # the cache is not in host memory (backend.h:66-68)

    def wait_kv_written(self, layer: int) -> None:
        _lib.check(self._L.rb200_wait_kv_written(self._h, layer))

    def update_weight(self, name: str, src, n: Optional[int] = None) -> None:
        """`src`: a float32 numpy array, or a raw address (host or any GPU) with `n` elements."""
        if isinstance(src, np.ndarray):
            a = np.ascontiguousarray(src, dtype=np.float32)
            _lib.check(self._L.rb200_update_weight(self._h, name.encode(), ptr(a), a.size))
        else:
            _lib.check(self._L.rb200_update_weight(self._h, name.encode(), C.c_void_p(int(src)), int(n)))

    # -- measurement support ------------------------------------------------------------------
    def set_profiling(self, on: bool) -> None:
        _lib.check(self._L.rb200_set_profiling(self._h, int(on)))

    def take_profile(self) -> dict:
        p = _lib.CProfile()
        _lib.check(self._L.rb200_get_profile(self._h, C.byref(p)))
        return {k: getattr(p, k) for k, _ in p._fields_}

    def forward_replay(self, iters: int) -> float:
        """Device milliseconds of `iters` re-runs of the last forward pass's kernels."""
        ms = C.c_float(0)
        _lib.check(self._L.rb200_forward_replay(self._h, iters, C.byref(ms)))
        return ms.value

    def debug_fill_kv(self, seed: int) -> None:
        _lib.check(self._L.rb200_debug_fill_kv(self._h, seed))

    # -- the NCCL KV hop ----------------------------------------------------------------------
    @staticmethod
    def nccl_unique_id() -> bytes:
        buf = C.create_string_buffer(_lib.NCCL_ID_BYTES)
        _lib.check(_lib.lib().rb200_nccl_unique_id(buf))
        return buf.raw

    def nccl_init(self, uid: bytes, nranks: int, rank: int) -> None:
        _lib.check(self._L.rb200_nccl_init(self._h, C.c_char_p(uid), nranks, rank))

    def nccl_finalize(self) -> None:
        _lib.check(self._L.rb200_nccl_finalize(self._h))

    def send_kv_layer(self, peer: int, layer: int, blocks: Sequence[int]) -> None:
        b = i32(blocks)
        _lib.check(self._L.rb200_send_kv_layer(self._h, peer, layer, ptr(b), b.size))

    def recv_kv_layer(self, peer: int, layer: int, blocks: Sequence[int]) -> None:
        b = i32(blocks)
        _lib.check(self._L.rb200_recv_kv_layer(self._h, peer, layer, ptr(b), b.size))

    # -- K/V links (plain peer stores + counters; include/relay_b200.h) ------------------------
    def kv_link_create(self, n_slots: int, slot_bytes: int) -> Tuple[int, bytes]:
        """(link id, handle to give to the other end)."""
        buf = C.create_string_buffer(_lib.KV_LINK_HANDLE_BYTES)
        link = _lib.check(self._L.rb200_kv_link_create(self._h, n_slots, slot_bytes, buf))
        return link, buf.raw

    def kv_link_connect(self, link: int, peer_handle: bytes) -> None:
        _lib.check(self._L.rb200_kv_link_connect(self._h, link, C.c_char_p(peer_handle)))

    def kv_link_send_layer(self, link: int, layer: int, blocks: Sequence[int]) -> None:
        b = i32(blocks)
        _lib.check(self._L.rb200_kv_link_send_layer(self._h, link, layer, ptr(b), b.size))

    def kv_link_recv_layer(self, link: int, layer: int, blocks: Sequence[int]) -> None:
        b = i32(blocks)
        _lib.check(self._L.rb200_kv_link_recv_layer(self._h, link, layer, ptr(b), b.size))

    def kv_link_send_layers(self, link: int, first_layer: int, n_layers: int, blocks: Sequence[int]) -> None:
        """Consecutive layers of a finished request, as many per message as a slot holds."""
        b = i32(blocks)
        _lib.check(self._L.rb200_kv_link_send_layers(self._h, link, first_layer, n_layers, ptr(b), b.size))

    def kv_link_recv_layers(self, link: int, first_layer: int, n_layers: int, blocks: Sequence[int]) -> None:
        b = i32(blocks)
        _lib.check(self._L.rb200_kv_link_recv_layers(self._h, link, first_layer, n_layers, ptr(b), b.size))

    def kv_link_skip_layers(self, link: int, n_layers: int, n_blocks: int) -> None:
        _lib.check(self._L.rb200_kv_link_skip_layers(self._h, link, n_layers, n_blocks))

    @staticmethod
    def kv_link_plan(slot_bytes: int, block_bytes: int, n_layers: int, n_blocks: int) -> Tuple[int, int]:
        """(messages, most whole layers in one message) for such a request over a ring of such slots."""
        per = C.c_int32(0)
        n = _lib.lib().rb200_kv_link_plan(slot_bytes, block_bytes, n_layers, n_blocks, C.byref(per))
        if n < 0:
            raise ValueError("kv_link_plan: arguments no link accepts")
        return n, per.value

    def kv_link_connect_local(self, link: int, other: "Backend", other_link: int) -> None:
        """Joins two backends of this process (same or different devices) by address."""
        _lib.check(self._L.rb200_kv_link_connect_local(self._h, link, other._h, other_link))

    def kv_link_wait(self, link: int, timeout_ms: int = 0) -> None:
        _lib.check(self._L.rb200_kv_link_wait(self._h, link, timeout_ms))

    def kv_link_close(self, link: int) -> None:
        _lib.check(self._L.rb200_kv_link_close(self._h, link))

    def kv_hop_sync(self, timeout_ms: int = 0) -> None:
        _lib.check(self._L.rb200_kv_hop_sync(self._h, timeout_ms))


def make_cuda_backend(weights: HostWeights, num_blocks: int, block_size: int, device: int = 0,
                      max_batch_tokens: int = 1024, max_context: Optional[int] = None,
                      options: Optional[CudaOptions] = None) -> Backend:
    """relay::make_cuda_backend (engine/include/relay/backend.h:95-97)."""
    return Backend(weights.config, weights, num_blocks, block_size, device, max_batch_tokens, max_context, options)
