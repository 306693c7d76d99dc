"""Loads ``libsrlm_kernels.so`` and wraps each exported kernel for torch tensors.

There is no other implementation behind these functions: if the library cannot
be built or loaded, or a tensor is not on a CUDA device, the call raises.
Tensors are passed as raw device pointers; every launch goes to torch's
current stream, so the calls can be recorded into a CUDA graph.
"""
from __future__ import annotations

import ctypes as C
import functools
from typing import Optional

import torch

from ..errors import ShapeError, Unavailable

DT_F32, DT_BF16 = 0, 1
_CODES = {torch.float32: DT_F32, torch.bfloat16: DT_BF16}


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _CODES[dt]
    except KeyError:
        raise ShapeError(f"dtype {dt} is not taken by the kernels (float32 or bfloat16)") from None


def _ptr(t: Optional[torch.Tensor]):
    if t is None:
        return C.c_void_p(0)
    if not t.is_cuda:
        raise Unavailable("kernels take CUDA tensors only; there is no CPU path")
    if not t.is_contiguous():
        raise ShapeError("kernels take contiguous tensors")
    return C.c_void_p(t.data_ptr())


# torch.cuda.current_stream() builds a Stream object through several Python layers (3.4 us measured, a
# third of a launch's host cost); the two calls below are what it ends in.
_RAW_STREAM = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_CURRENT_DEVICE = getattr(torch._C, "_cuda_getDevice", None)


def _stream():
    """The current CUDA stream of the current device (the capturing one while a graph is recorded)."""
    if _RAW_STREAM is not None and _CURRENT_DEVICE is not None:
        return C.c_void_p(_RAW_STREAM(_CURRENT_DEVICE()))
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


class KernelLibrary:
    def __init__(self):
        self._lib = None
        self.launches = 0          # kernels launched through this object (a benchmark reports it)
        self.force_simt_gemm = False   # tests: run the float32 FMA twin in place of the tensor cores
        self.force_simt_attention = False
        self.force_tcgen05_gemm = False
        # The weight-streaming (mma.sync) kernel serves products of at most this many tokens and weight rows.
        # 0: none -- the one-tile tensor-core kernel with its K splits in a cluster streams the weights faster
        # at every token count (a layer's four products at 8 tokens: 70.8 against 82.8 us); 8 brings it back.
        self.skinny_max_tokens = 0
        self.skinny_max_rows = 1 << 30
        self.force_cp_async_decode = False
        self.cluster_decode_merge = True        # slices of decode attention merged in a thread-block cluster
        self.fuse_decode_attention = True       # decode: norm, rotation and append inside the attention kernel
        self.force_mma_sync_prefill = False
        self.split_mixed_attention = True       # mixed steps: decoding requests to the keys-split kernel ...
        self.split_prefill_keys = True          # rows-split attention: the keys in slices when rows are few
        self.split_mixed_min_blocks = None      # ... when they make this many blocks (None: one per SM)
        self.fuse_norms_into_products = True    # steps of up to 128 tokens: the blocks' norms inside the products
        self.early_launch = True                # weight-streaming products may start under the kernel ahead of them

    @property
    def lib(self):
        if self._lib is None:
            from ..csrc.build import build_kernels
            try:
                path = build_kernels()
                self._lib = C.CDLL(path)
            except Exception as e:   # noqa: BLE001
                raise Unavailable(f"the CUDA kernel library is missing and could not be built: {e}") from e
            self._lib.srlm_last_error.restype = C.c_char_p
            import os
            if os.environ.get("SRLM_PDL", "1") == "0":     # plain stream order between kernels
                self._lib.srlm_set_pdl(0)
        return self._lib

    def sm_count(self, device) -> int:
        counts = self.__dict__.setdefault("_sm_counts", {})
        if device not in counts:
            counts[device] = torch.cuda.get_device_properties(device).multi_processor_count
        return counts[device]

    def set_pdl(self, on: bool) -> None:
        """Programmatic dependent launch between the kernels of a step (on by default)."""
        self.lib.srlm_set_pdl(C.c_int(1 if on else 0))

    def begin_timing(self) -> None:
        """From now on every launch is followed by a CUDA event; ``end_timing`` turns the gaps between
        consecutive events into a table.  Kernels of one stream run one after the other, so the gap
        before a launch's event is that kernel's time (with its launch gap; no overlap between kernels
        is possible while this is on: use it on eager steps, for shares, not for absolutes; launches that
        go into a CUDA graph under capture are left out)."""
        start = torch.cuda.Event(enable_timing=True)
        start.record()
        self._timing = [("", start)]

    def end_timing(self) -> dict:
        """{kernel name: (launches, milliseconds)} since begin_timing (waits for the device)."""
        marks, self._timing = getattr(self, "_timing", None) or [], None
        torch.cuda.synchronize()
        table: dict = {}
        for (_, before), (name, after) in zip(marks, marks[1:]):
            n, ms = table.get(name, (0, 0.0))
            table[name] = (n + 1, ms + before.elapsed_time(after))
        return table

    def _check(self, status: int, what: str):
        self.launches += 1
        if getattr(self, "_timing", None) is not None and status == 0 \
                and not torch.cuda.is_current_stream_capturing():      # a timed event cannot be recorded into a graph
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self._timing.append((what, ev))
        if status != 0:
            msg = self.lib.srlm_last_error().decode(errors="replace")
            if status < 0:
                raise ShapeError(f"{what} refused: {msg}")
            raise RuntimeError(f"{what} failed with CUDA error {status}: {msg}")

    # ---- elementwise -----------------------------------------------------
    def embed_gather(self, ids, table, out, bad_flag):
        T, H = out.shape
        self._check(self.lib.srlm_embed_gather(_ptr(ids), _ptr(table), dtype_code(table.dtype), _ptr(out),
                                               C.c_int(T), C.c_int(H), C.c_int(table.shape[0]),
                                               _ptr(bad_flag), _stream()), "embed_gather")

    def add_rmsnorm(self, residual, delta, weight, eps, out, rows=None, unit_offset=False):
        R, H = out.shape
        self._check(self.lib.srlm_add_rmsnorm(_ptr(residual), _ptr(delta), _ptr(weight), C.c_float(eps),
                                              _ptr(out), dtype_code(out.dtype), _ptr(rows), C.c_int(R),
                                              C.c_int(H), C.c_int(int(unit_offset)), _stream()),
                    "add_rmsnorm")

    def swiglu(self, gate_up, out):
        T, I = out.shape
        self._check(self.lib.srlm_swiglu(_ptr(gate_up), _ptr(out), dtype_code(out.dtype), C.c_int(T),
                                         C.c_int(I), _stream()), "swiglu")

    def cast(self, src, dst):
        self._check(self.lib.srlm_cast(_ptr(src), dtype_code(src.dtype), _ptr(dst), dtype_code(dst.dtype),
                                       C.c_longlong(src.numel()), _stream()), "cast")

    def patch_words(self, words, pairs, src, n, flag):
        """words[pairs[2 i]] = src[pairs[2 i + 1]] for i < n, all int32 on the device: token ids that a step
        takes from what the step before it sampled, before the host has read them.  An index outside its
        tensor is skipped and raises flag[0]."""
        if any(t.dtype != torch.int32 for t in (words, pairs, src, flag)) or pairs.numel() < 2 * n:
            raise ShapeError("patch_words: int32 tensors, two words a pair")
        self._check(self.lib.srlm_patch_words(_ptr(words), C.c_longlong(words.numel()), _ptr(pairs), _ptr(src),
                                              C.c_int(src.numel()), C.c_int(n), _ptr(flag), _stream()), "patch_words")

    def check_finite(self, a, b, flag):
        """flag[0] = 1 if any element of a (+ b, same shape, when given) is NaN or infinite; a float32."""
        if a.dtype != torch.float32 or (b is not None and b.numel() != a.numel()):
            raise ShapeError("check_finite: a must be float32 and b of the same size")
        self._check(self.lib.srlm_check_finite(_ptr(a), _ptr(b), dtype_code(b.dtype) if b is not None else DT_F32,
                                               C.c_longlong(a.numel()), _ptr(flag), _stream()), "check_finite")

    def residual_add(self, residual, delta):
        self._check(self.lib.srlm_residual_add(_ptr(residual), _ptr(delta), dtype_code(delta.dtype),
                                               C.c_longlong(delta.numel()), _stream()), "residual_add")

    # ---- position encoding and cache append ------------------------------
    def rope_table(self, positions, cos, sin, theta, rotary_dim):
        T, half = cos.shape
        self._check(self.lib.srlm_rope_table(_ptr(positions), _ptr(cos), _ptr(sin), C.c_int(T), C.c_int(half),
                                             C.c_double(theta), C.c_int(rotary_dim), _stream()), "rope_table")

    def qk_norm_rope_append(self, qkv, q_out, k_cache, v_cache, q_norm_w, k_norm_w, eps, cos, sin, kv_slot,
                            nq, nkv, hd, rotary_half, write_kv=True, interleaved=False):
        """k_cache / v_cache: [pages, kv_heads, page_size, head_dim]; kv_slot[t] = page * page_size + offset.
        cos / sin [T, rotary_half] rotate the pairs (i, i + rotary_half), or (2i, 2i + 1) when interleaved,
        of the first 2 * rotary_half elements of every q and k head; rotary_half 0: no rotation."""
        T = qkv.shape[0]
        self._check(self.lib.srlm_qk_norm_rope_append(
            _ptr(qkv), _ptr(q_out), dtype_code(qkv.dtype), _ptr(k_cache), _ptr(v_cache),
            dtype_code(k_cache.dtype), _ptr(q_norm_w), _ptr(k_norm_w), C.c_float(eps), _ptr(cos), _ptr(sin),
            _ptr(kv_slot), C.c_int(T), C.c_int(nq), C.c_int(nkv), C.c_int(hd), C.c_int(rotary_half),
            C.c_int(int(write_kv)), C.c_int(k_cache.shape[2]), C.c_int(int(interleaved)), _stream()),
            "qk_norm_rope_append")

    # ---- attention --------------------------------------------------------
    def paged_attention_simt(self, q, k_cache, v_cache, out, block_table, entry_of_token, positions,
                             nq, nkv, hd, page_size, scale, window=0):
        T = q.shape[0]
        self._check(self.lib.srlm_paged_attention_simt(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), dtype_code(q.dtype), dtype_code(k_cache.dtype),
            _ptr(block_table), C.c_int(block_table.stride(0)), _ptr(entry_of_token), _ptr(positions),
            C.c_int(T), C.c_int(nq), C.c_int(nkv), C.c_int(hd), C.c_int(page_size), C.c_float(scale),
            C.c_int(window or 0), _stream()), "paged_attention_simt")

    # ---- matrix products ----------------------------------------------------
    def gemm_tn_simt(self, a, w, out):
        """out[M,N] = a[M,K] @ w[N,K]^T, float32 FMA accumulation."""
        M, K = a.shape
        N = w.shape[0]
        if w.shape[1] != K or tuple(out.shape) != (M, N):
            raise ShapeError(f"gemm: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
        self._check(self.lib.srlm_gemm_tn_simt(
            _ptr(a), dtype_code(a.dtype), _ptr(w), dtype_code(w.dtype), _ptr(out), dtype_code(out.dtype),
            C.c_int(M), C.c_int(N), C.c_int(K), C.c_longlong(a.stride(0)), C.c_longlong(w.stride(0)),
            C.c_longlong(out.stride(0)), _stream()), "gemm_tn_simt")

    # split-K workspace of the tensor-core GEMM: 64 KiB of tile counters, then float32 partials
    GEMM_WS_BYTES = 65536 + (64 << 20)

    def _gemm_state(self, device):
        st = getattr(self, "_gemm_ws", None)
        if st is None or st[0].device != device:
            ws = torch.zeros(self.GEMM_WS_BYTES, dtype=torch.uint8, device=device)
            err = torch.zeros(1, dtype=torch.int32, device=device)
            st = self._gemm_ws = (ws, err)
        bound = getattr(self, "_bound_err", None)
        if bound is not None and bound.device == device:
            return st[0], bound
        return st

    def bind_error_flag(self, flag: Optional[torch.Tensor]) -> None:
        """The int32 word that kernels with bounded waits (TMA / tensor-core pipelines) raise when a wait
        runs out.  An engine binds a word of its own status buffer before each forward, so that the
        step's read-back sees it; None goes back to the library's own word."""
        self._bound_err = flag

    def wait_probe(self, flag: torch.Tensor, limit_cycles: int = 1_000_000, code: int = 99) -> None:
        """A kernel whose one bounded wait (the pipelines' own, on a barrier nobody arrives at) runs out after
        ``limit_cycles`` and writes ``code`` to flag[0], then ends normally.  For tests of the way from such a
        wait to the host; the product path never launches it."""
        if flag.dtype != torch.int32:
            raise ShapeError("wait_probe: an int32 flag")
        self._check(self.lib.srlm_wait_probe(_ptr(flag), C.c_longlong(limit_cycles), C.c_int(code), _stream()),
                    "wait_probe")

    def gemm_error_flag(self, device) -> int:
        """Nonzero if a kernel gave up on a bounded wait since the flag was last read (synchronises)."""
        err = self._gemm_state(device)[1]
        v = int(err.item())
        if v:
            err.zero_()
        return v

    # The plans below are made on the host, also where there is no GPU (tests).  They are tuned for the
    # B200's 148 SMs, and the token-tile rule repeats the one in gemm_tcgen05.cu
    # (srlm_gemm_tcgen05_token_tile reports the kernel's own choice; a GPU test holds the two together).
    SMS = 148
    BN256_MIN_TILES = 96

    @staticmethod
    @functools.lru_cache(maxsize=4096)
    def gemm_token_tile(M: int, N: int) -> int:
        """The width of the token tiles of the tensor-core product of M tokens and N weight rows (the rule
        of token_tile in gemm_tcgen05.cu, where its reasons and measurements stand)."""
        if M <= 128:
            return 16 if M <= 16 else 32 if M <= 32 else 64 if M <= 64 else 128
        rows128 = (N + 127) // 128
        if rows128 * ((M + 255) // 256) >= KernelLibrary.BN256_MIN_TILES:
            return 256
        sms = KernelLibrary.SMS
        tiles128, tiles256 = rows128 * ((M + 127) // 128), ((N + 255) // 256) * ((M + 255) // 256)
        rounds128, rounds256 = -(-tiles128 // sms), -(-tiles256 // (sms // 2))
        return 256 if 4 * rounds256 < 3 * rounds128 else 128

    @staticmethod
    @functools.lru_cache(maxsize=4096)
    def gemm_splits(M: int, N: int, K: int) -> int:
        """How many ways to split K: the number of blocks should fill whole waves of the SMs
        (192 tiles alone would leave the second wave two thirds empty), each split keeping at
        least 4 k-blocks, the partial sums fitting the workspace."""
        bn = KernelLibrary.gemm_token_tile(M, N)
        if bn == 256:
            return 1                      # pairs of SMs on whole tiles of 256 x 256
        tiles = ((N + 127) // 128) * ((M + bn - 1) // bn)
        total_kb = (K + 63) // 64
        if tiles >= 1024:
            return 1
        if M > 16:
            # Measured on B200, 8B layer sizes: splitting until about 200 blocks stream (a few more up to 32
            # tokens) pays, each split keeping at least 8 k-blocks.  Up to 8 splits add their sums inside a
            # thread-block cluster; with that, 4 splits also pay from 65 to a few hundred tokens, where
            # an unsplit product of a narrow output leaves most SMs without a tile (128 tokens: o and down
            # projections 27.6 -> 21.5 us and 64.5 -> 35.6 us).
            if M <= 32:
                sp = min(222 // max(1, tiles), total_kb // 8)
            elif M <= 64:
                sp = min(200 // max(1, tiles), total_kb // 8, 8)
            else:
                # tiles of 128 tokens, two blocks to an SM: up to about 256 blocks run as one round (clusters
                # of 3 or 4 do not pack the GPCs to the last slot: 288 blocks measured a round more).  At 256
                # tokens, 14B sizes: down projection 61.5 -> 53.3 us with 3 splits instead of 2 (80 tiles),
                # 8B sizes: 36.1 -> 31.3 us with 4 instead of 3 (64 tiles); 512 tokens, 8B: 58.4 -> 51.8 us
                # with 2 splits of 128 tiles
                sp = min(256 // max(1, tiles), total_kb // 8, 4)
                if M <= 128:
                    # one token tile: a long K pays more splits (down projection of 128 tokens, 4096 x 12,288:
                    # 28.5 us in 4 splits, 25.6 in 6, 24.3 in 8; the output projection's K of 4096 does not)
                    sp = max(sp, min(256 // max(1, tiles), total_kb // 16, 8))
            sp = max(1, sp)
            if M <= 64 and sp == 1 and 148 < tiles and 2 * tiles <= 444 and total_kb >= 16:
                sp = 2        # three blocks of a shallower ring an SM (the kernel picks it by the block count)
            while sp > 8 and 65536 + sp * tiles * 128 * bn * 4 > KernelLibrary.GEMM_WS_BYTES:
                sp -= 1
            return sp
        # Up to 16 tokens three blocks share an SM (444 at a time); splits up to the cluster's 8.  Measured on
        # B200 at 16 tokens, 8B layer sizes (QKV / O / gate-up / down): 4-8 / 6-8 / 2 / 6-8 splits are best
        # (11.6 / 9.6 / 32.1 / 19.7 us; gate/up unsplit 35.0 us, in 3 splits 37.5 us; down in 9 splits through
        # the workspace 23.4 us).
        return max(1, min(444 // max(1, tiles), total_kb // 8, 8))

    def gemm_tn_tcgen05(self, a, w, out, splits=None, swiglu8=False):
        """out[M,N] = a[M,K] @ w[N,K]^T, bfloat16 operands, tcgen05 tensor cores, float32 accumulation.
        swiglu8: w's rows come in blocks of 16 (8 gate rows, then the 8 up rows of the same features)
        and out[M, N/2] = silu(gate) * up."""
        M, K = a.shape
        N = w.shape[0]
        if (w.shape[1] != K or tuple(out.shape) != (M, N // 2 if swiglu8 else N) or a.dtype != torch.bfloat16
                or w.dtype != torch.bfloat16):
            raise ShapeError(f"gemm_tcgen05: a {tuple(a.shape)} {a.dtype}, w {tuple(w.shape)} {w.dtype}, "
                             f"out {tuple(out.shape)}")
        ws, err = self._gemm_state(a.device)
        if splits is None:
            splits = self.gemm_splits(M, N, K)
        self._check(self.lib.srlm_gemm_tn_tcgen05(
            _ptr(a), _ptr(w), _ptr(out), dtype_code(out.dtype), C.c_int(M), C.c_int(N), C.c_int(K),
            C.c_longlong(a.stride(0)), C.c_longlong(w.stride(0)), C.c_longlong(out.stride(0)), C.c_int(splits),
            _ptr(ws), C.c_longlong(ws.numel()), _ptr(err), C.c_int(int(swiglu8)), _stream()),
            f"gemm_tn_tcgen05[{M}x{N}x{K}]" if getattr(self, "_timing", None) is not None else "gemm_tn_tcgen05")

    FUSED_TOKENS = 128       # most tokens of a product that runs its norms inside itself

    def gemm_tn_tcgen05_fused(self, a, w, out=None, swiglu8=False, scale_parts=None, norm_width=0, eps=0.0,
                              residual=None, next_w=None, xw_out=None, ss_out=None):
        """The tensor-core product of at most 128 tokens fused with the norms around it: the same contract
        as gemm_tn_skinny_fused, except that the partial sums of squares lie as [parts, tokens]
        (scale_parts: any row stride; ss_out: [ceil(N / 128), >= M])."""
        M, K = a.shape
        N = w.shape[0]
        if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.shape[1] != K or M > self.FUSED_TOKENS:
            raise ShapeError(f"gemm_tcgen05_fused: a {tuple(a.shape)} {a.dtype}, w {tuple(w.shape)} {w.dtype}")
        if residual is None and (out is None or tuple(out.shape) != (M, N // 2 if swiglu8 else N)):
            raise ShapeError("gemm_tcgen05_fused: out has the wrong shape")
        if ss_out is not None and (ss_out.shape[0] < (N + 127) // 128 or ss_out.shape[1] < M):
            raise ShapeError("gemm_tcgen05_fused: ss_out must be [ceil(N/128), >= M]")
        ws, err = self._gemm_state(a.device)
        self._check(self.lib.srlm_gemm_tn_tcgen05_fused(
            _ptr(a), _ptr(w), _ptr(out), dtype_code(out.dtype) if out is not None else DT_BF16, C.c_int(M),
            C.c_int(N), C.c_int(K), C.c_longlong(a.stride(0)), C.c_longlong(w.stride(0)),
            C.c_longlong(out.stride(0) if out is not None else N), C.c_int(self.gemm_splits(M, N, K)), _ptr(ws),
            C.c_longlong(ws.numel()), _ptr(err), C.c_int(int(swiglu8)), _ptr(scale_parts),
            C.c_int(scale_parts.shape[0] if scale_parts is not None else 0),
            C.c_longlong(scale_parts.stride(0) if scale_parts is not None else 0), C.c_int(norm_width), C.c_float(eps),
            _ptr(residual), C.c_longlong(residual.stride(0) if residual is not None else 0), _ptr(next_w),
            _ptr(xw_out), C.c_longlong(xw_out.stride(0) if xw_out is not None else 0), _ptr(ss_out),
            C.c_longlong(ss_out.stride(0) if ss_out is not None else 0), _stream()),
            f"gemm_tn_tcgen05_fused[{M}x{N}x{K}]" if getattr(self, "_timing", None) is not None
            else "gemm_tn_tcgen05_fused")

    def gemm_dealt_tiles(self, M: int, N: int, K: int) -> int:
        """How many tiles of this product the persistent tensor-core kernel deals out by k-blocks
        (0: whole tiles only, or another kernel serves these sizes)."""
        return int(self.lib.srlm_gemm_tcgen05_dealt_tiles(C.c_int(M), C.c_int(N), C.c_int(K)))

    def gemm_tn_skinny(self, a, w, out, swiglu8=False, early=True):
        """out[M,N] = a[M,K] @ w[N,K]^T for M <= 16: the weight-streaming kernel of decode steps.
        swiglu8: as in gemm_tn_tcgen05.  early: the kernel may start under the tail of the kernel ahead
        of it (it requests its first weights, then waits for that kernel's results); False for the
        product that follows a mixer's own kernel, where that measured much slower."""
        M, K = a.shape
        N = w.shape[0]
        if (w.shape[1] != K or tuple(out.shape) != (M, N // 2 if swiglu8 else N) or a.dtype != torch.bfloat16
                or w.dtype != torch.bfloat16):
            raise ShapeError(f"gemm_skinny: a {tuple(a.shape)} {a.dtype}, w {tuple(w.shape)} {w.dtype}, "
                             f"out {tuple(out.shape)}")
        self._check(self.lib.srlm_gemm_tn_skinny(
            _ptr(a), _ptr(w), _ptr(out), dtype_code(out.dtype), C.c_int(M), C.c_int(N), C.c_int(K),
            C.c_longlong(a.stride(0)), C.c_longlong(w.stride(0)), C.c_longlong(out.stride(0)),
            C.c_int(int(swiglu8)), C.c_int(int(early and self.early_launch)), _stream()),
            f"gemm_tn_skinny[{M}x{N}x{K}]" if getattr(self, "_timing", None) is not None else "gemm_tn_skinny")

    def gemm_tn_skinny_fused(self, a, w, out=None, swiglu8=False, scale_parts=None, norm_width=0, eps=0.0,
                             residual=None, next_w=None, xw_out=None, ss_out=None, early=True):
        """The weight-streaming product (at most 8 tokens) fused with the norms around it.

        scale_parts [parts, 8] float32: ``a`` holds bf16(residual * norm weight); the product is scaled per
        token by rsqrt(sum of the parts / norm_width + eps).  residual [M, N] float32: the product is added
        to it in place instead of being stored; with next_w [N] also xw_out[M, N] = bf16(residual * next_w)
        and ss_out [N/16, 8] (each block's share of the rows' sums of squares) are written."""
        M, K = a.shape
        N = w.shape[0]
        if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.shape[1] != K or M > 8:
            raise ShapeError(f"gemm_skinny_fused: a {tuple(a.shape)} {a.dtype}, w {tuple(w.shape)} {w.dtype}")
        if residual is None and (out is None or tuple(out.shape) != (M, N // 2 if swiglu8 else N)):
            raise ShapeError("gemm_skinny_fused: out has the wrong shape")
        if ss_out is not None and (ss_out.shape[0] < (N + 15) // 16 or ss_out.shape[1] != 8):
            raise ShapeError("gemm_skinny_fused: ss_out must be [ceil(N/16), 8]")
        self._check(self.lib.srlm_gemm_tn_skinny_fused(
            _ptr(a), _ptr(w), _ptr(out), dtype_code(out.dtype) if out is not None else DT_BF16, C.c_int(M),
            C.c_int(N), C.c_int(K), C.c_longlong(a.stride(0)), C.c_longlong(w.stride(0)),
            C.c_longlong(out.stride(0) if out is not None else N), C.c_int(int(swiglu8)), _ptr(scale_parts),
            C.c_int(scale_parts.shape[0] if scale_parts is not None else 0), C.c_int(norm_width), C.c_float(eps),
            _ptr(residual), C.c_longlong(residual.stride(0) if residual is not None else 0), _ptr(next_w),
            _ptr(xw_out), C.c_longlong(xw_out.stride(0) if xw_out is not None else 0), _ptr(ss_out),
            C.c_int(int(early and self.early_launch)), _stream()),
            f"gemm_tn_skinny_fused[{M}x{N}x{K}]" if getattr(self, "_timing", None) is not None
            else "gemm_tn_skinny_fused")

    def fuses_in_skinny(self, T: int, w) -> bool:
        """Whether a fused product of T tokens runs the weight-streaming kernel (else the tensor-core one)."""
        return T <= min(8, self.skinny_max_tokens) and w.shape[0] <= self.skinny_max_rows \
            and not self.force_tcgen05_gemm

    def can_fuse_norms(self, T: int, dtype, w) -> bool:
        """Whether a product of T tokens with this weight may run the norms around it inside itself: the
        weight-streaming kernel up to 8 tokens, the one-tile tensor-core kernel up to 128."""
        return (dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and T <= self.FUSED_TOKENS
                and w.shape[1] % 8 == 0 and not self.force_simt_gemm and self.fuse_norms_into_products)

    def can_fuse_swiglu(self, a_dtype, w) -> bool:
        """Whether gemm(..., swiglu8=True) is offered for these operands (the tensor-core kernels only)."""
        return (a_dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[1] % 8 == 0
                and w.shape[0] % 16 == 0 and not self.force_simt_gemm)

    def gemm(self, a, w, out, swiglu8=False, early=True):
        """The product path's matrix product: picks the kernel for the dtypes and sizes.  bfloat16
        operands go to the tensor cores; float32 operands, and widths that TMA cannot address
        (K not a multiple of 8), go to the float32 FMA kernel.  early: see gemm_tn_skinny."""
        if (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.shape[1] % 8 == 0
                and not self.force_simt_gemm):
            if a.shape[0] <= self.skinny_max_tokens and w.shape[0] <= self.skinny_max_rows \
                    and not self.force_tcgen05_gemm:
                self.gemm_tn_skinny(a, w, out, swiglu8, early=early)   # a few tokens: bound by streaming the weights
            else:
                self.gemm_tn_tcgen05(a, w, out, swiglu8=swiglu8)
        else:
            if swiglu8:
                raise ShapeError("the fused SwiGLU epilogue exists in the bfloat16 tensor-core kernels only")
            self.gemm_tn_simt(a, w, out)

    def paged_attention_rows(self, q, k_cache, v_cache, out, block_table, cu_q, kv_lens, work, nq, nkv, hd,
                             page_size, scale, window=0):
        """bfloat16 tensor-core attention for a ragged batch; work: int32 [n, 2] (entry, tile of 64 rows)."""
        self._check(self.lib.srlm_paged_attention_rows(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(block_table), C.c_int(block_table.stride(0)),
            _ptr(cu_q), _ptr(kv_lens), _ptr(work), C.c_int(work.shape[0]), C.c_int(nq), C.c_int(nkv), C.c_int(hd),
            C.c_int(page_size), C.c_float(scale), C.c_int(window or 0), _stream()), "paged_attention_rows")

    def paged_attention_rows_tma(self, q, k_cache, v_cache, out, block_table, cu_q, kv_lens, work, nq, nkv, hd,
                                 page_size, scale, window=0):
        """Rows-split attention with TMA page loads; work: int32 [n, 2] (entry, tile of 128 rows)."""
        err = self._gemm_state(q.device)[1]
        self._check(self.lib.srlm_paged_attention_rows_tma(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), C.c_longlong(k_cache.shape[0]), _ptr(block_table),
            C.c_int(block_table.stride(0)), _ptr(cu_q), _ptr(kv_lens), _ptr(work), C.c_int(work.shape[0]),
            C.c_int(nq), C.c_int(nkv), C.c_int(hd), C.c_int(page_size), C.c_float(scale), C.c_int(window or 0),
            _ptr(err), _stream()), "paged_attention_rows_tma")

    def paged_attention_prefill_tcgen05(self, q, k_cache, v_cache, out, block_table, cu_q, kv_lens, work, nq, nkv,
                                        hd, page_size, scale, window=0, tiles_per_block=2, nsplit=1, kv_chunk=0,
                                        part_o=None, part_ml=None):
        """Rows-split attention on tcgen05 tensor cores with accumulators in tensor memory (head size
        128; page_size 8..64 a power of two, or a multiple of 128); work: int32 [n, 2] (entry, block of
        tiles_per_block x 128 rows), tiles_per_block 1 or 2.  nsplit > 1: the keys in slices of kv_chunk
        (a multiple of 128), a block each, added by a second kernel; part_o float32
        [n * 2 * nkv * nsplit * 128, 128] and part_ml [.., 2] are their workspace."""
        err = self._gemm_state(q.device)[1]
        self._check(self.lib.srlm_paged_attention_prefill_tcgen05(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), C.c_longlong(k_cache.shape[0]), _ptr(block_table),
            C.c_int(block_table.stride(0)), _ptr(cu_q), _ptr(kv_lens), _ptr(work), C.c_int(work.shape[0]),
            C.c_int(nq), C.c_int(nkv), C.c_int(hd), C.c_int(page_size), C.c_float(scale), C.c_int(window or 0),
            C.c_int(tiles_per_block), C.c_int(nsplit), C.c_int(kv_chunk), _ptr(part_o), _ptr(part_ml), _ptr(err),
            _stream()), "paged_attention_prefill_tcgen05")
        if nsplit > 1:
            self.launches += 1           # the kernel that adds the slices

    @staticmethod
    def prefill_attention_plan(rows, kv_lens, nkv: int, sms: int):
        """(tiles_per_block, nsplit, kv_chunk) for the tensor-memory attention kernel on entries of
        ``rows`` rows (tokens x query heads per KV head) and ``kv_lens`` keys.  The choice goes by a
        model of the kernel's time, fitted to measurements on B200 (one portion of 481 to 512 tokens behind
        1,024 and 8,192 cached ones, 32 and 40 heads over 8 KV heads), in microseconds: a block of one row
        tile takes 7.8 + 1.75 a key tile, a block of two row tiles 11.7 + 1.92 a key tile (the tensor core
        works on one tile while the other is in its softmax), blocks run in rounds of one per SM, and
        cutting the keys into slices adds 11 (the slices' outputs go through a workspace and a second
        kernel).  So: two row tiles a block when the rows fill the SMs or one-tile blocks would need a
        round more; key slices for a portion behind a long context (512 tokens behind 8,192: 126.6 us in
        one-tile blocks, 88.6 us in two slices of two-tile blocks)."""
        two_tile_blocks = sum((r + 255) // 256 for r in rows) * nkv
        one_tile_blocks = sum((r + 127) // 128 for r in rows) * nkv
        key_tiles = max(1, (max(kv_lens) + 127) // 128)
        rounds = lambda blocks: -(-blocks // max(1, sms))
        best = (rounds(one_tile_blocks) * (key_tiles * 1.75 + 7.8), 1, 1)
        for s in range(1, min(16, max(1, key_tiles // 2)) + 1):
            per_slice = -(-key_tiles // s)
            t = rounds(two_tile_blocks * s) * (per_slice * 1.92 + 11.7) + (11.0 if s > 1 else 0.0)
            if t < best[0] - 1e-9:
                best = (t, 2, s)
        _, tiles, s = best
        if s == 1:
            return tiles, 1, 0
        chunk = -(-key_tiles // s) * 128
        return tiles, -(-key_tiles * 128 // chunk), chunk

    def paged_attention_keys(self, q, k_cache, v_cache, out, block_table, cu_q, kv_lens, n_entries, nq, nkv, hd,
                             page_size, scale, window, kv_chunk, nsplit, part_o=None, part_ml=None):
        """bfloat16 tensor-core attention when every entry has at most 16 rows (decode); keys in nsplit slices."""
        counters = None
        if nsplit > 1:
            counters = getattr(self, "_slice_counters", None)
            if counters is None or counters.device != q.device:
                counters = self._slice_counters = torch.zeros(1 << 16, dtype=torch.int32, device=q.device)
            if n_entries * nkv > counters.numel():
                raise ShapeError(f"paged_attention_keys: {n_entries} entries x {nkv} KV heads exceed the counters")
        self._check(self.lib.srlm_paged_attention_keys(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(block_table), C.c_int(block_table.stride(0)),
            _ptr(cu_q), _ptr(kv_lens), C.c_int(n_entries), C.c_int(nq), C.c_int(nkv), C.c_int(hd),
            C.c_int(page_size), C.c_float(scale), C.c_int(window or 0), C.c_int(kv_chunk), C.c_int(nsplit),
            _ptr(part_o), _ptr(part_ml), _ptr(counters), _stream()), "paged_attention_keys")

    def _slice_counter_buffer(self, device, need):
        counters = getattr(self, "_slice_counters", None)
        if counters is None or counters.device != device:
            counters = self._slice_counters = torch.zeros(1 << 16, dtype=torch.int32, device=device)
        if need > counters.numel():
            raise ShapeError(f"attention: {need} (entry, KV head) pairs exceed the slice counters")
        return counters

    def paged_attention_decode_tma(self, q, k_cache, v_cache, out, block_table, cu_q, kv_lens, n_entries, nq, nkv,
                                   hd, page_size, scale, window, kv_chunk, nsplit, part_o=None, part_ml=None,
                                   cluster=True):
        """Decode attention with TMA page loads (head_dim a multiple of 64; page_size 8, 16, 32 or a
        multiple of 64); same contract as paged_attention_keys.  cluster: up to 8 slices are merged
        through the distributed shared memory of a thread-block cluster (part_o / part_ml not needed)."""
        counters = self._slice_counter_buffer(q.device, n_entries * nkv) if nsplit > 1 else None
        err = self._gemm_state(q.device)[1]
        self._check(self.lib.srlm_paged_attention_decode_tma(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), C.c_longlong(k_cache.shape[0]), _ptr(block_table),
            C.c_int(block_table.stride(0)), _ptr(cu_q), _ptr(kv_lens), C.c_int(n_entries), C.c_int(nq),
            C.c_int(nkv), C.c_int(hd), C.c_int(page_size), C.c_float(scale), C.c_int(window or 0),
            C.c_int(kv_chunk), C.c_int(nsplit), _ptr(part_o), _ptr(part_ml), _ptr(counters),
            C.c_int(1 if cluster else 0), _ptr(err), _stream()), "paged_attention_decode_tma")

    def paged_attention_decode_fused(self, qkv, q_norm_w, k_norm_w, eps, cos, sin, write_kv, k_cache, v_cache, out,
                                     block_table, cu_q, kv_lens, n_entries, nq, nkv, hd, page_size, scale, window,
                                     kv_chunk, nsplit, part_o=None, part_ml=None, cluster=True):
        """paged_attention_decode_tma with the step before it folded in: q and the step's new keys and
        values are read from qkv [tokens, (nq + 2 nkv) * hd], normalised per head (weights may be None)
        and rotated (cos / sin [tokens, hd/2], pairs (i, i + hd/2)) inside the kernel; with write_kv the
        new keys and values are written to the cache.  head_dim 64, 128 or 256."""
        counters = self._slice_counter_buffer(qkv.device, n_entries * nkv) if nsplit > 1 else None
        err = self._gemm_state(qkv.device)[1]
        self._check(self.lib.srlm_paged_attention_decode_fused(
            _ptr(qkv), _ptr(q_norm_w), _ptr(k_norm_w), C.c_float(eps), _ptr(cos), _ptr(sin),
            C.c_int(int(write_kv)), _ptr(k_cache), _ptr(v_cache), _ptr(out), C.c_longlong(k_cache.shape[0]),
            _ptr(block_table), C.c_int(block_table.stride(0)), _ptr(cu_q), _ptr(kv_lens), C.c_int(n_entries),
            C.c_int(nq), C.c_int(nkv), C.c_int(hd), C.c_int(page_size), C.c_float(scale), C.c_int(window or 0),
            C.c_int(kv_chunk), C.c_int(nsplit), _ptr(part_o), _ptr(part_ml), _ptr(counters),
            C.c_int(1 if cluster else 0), _ptr(err), _stream()), "paged_attention_decode_fused")

    @staticmethod
    def attention_split(n_entries: int, nkv: int, max_kv: int, max_slices: int = 32):
        """(nsplit, kv_chunk) for the keys-split kernels: as many blocks as run at the same time (two per
        SM) and no more -- a few blocks left over for a second wave would double the time -- in slices of
        whole tiles."""
        tiles = max(1, (max_kv + 63) // 64)
        nsplit = max(1, min(tiles, 2 * KernelLibrary.SMS // max(1, n_entries * nkv), max_slices))
        chunk = -(-tiles // nsplit) * 64
        nsplit = -(-tiles * 64 // chunk)
        return nsplit, chunk

    def _decode_plan(self, ctx, nkv, hd, n_entries=None, kv_bound=None):
        """(nsplit, kv_chunk, cluster, part_o, part_ml) for the TMA decode kernel on the batch of ctx, or on
        ``n_entries`` of its entries whose keys number at most ``kv_bound``."""
        n_entries = ctx.n_entries if n_entries is None else n_entries
        kv_bound = ctx.kv_bound if kv_bound is None else kv_bound
        nsplit, chunk = self.attention_split(n_entries, nkv, kv_bound)
        # Up to 8 slices merge inside a thread-block cluster, which saves the round trip through global
        # memory (6 to 8 us measured); more slices pay only when each of the 8 would have many more
        # tiles to walk (about 1 us a tile).
        cluster = False
        if self.cluster_decode_merge and nsplit > 1:
            n8, chunk8 = self.attention_split(n_entries, nkv, kv_bound, max_slices=8)
            if chunk8 - chunk <= 7 * 64:
                nsplit, chunk, cluster = n8, chunk8, True
        part_o = part_ml = None
        if nsplit > 1 and not cluster:
            part_o = ctx.workspace.get("attn.part_o", n_entries * nkv * nsplit * 16, hd, torch.float32, reserve=0)
            part_ml = ctx.workspace.get("attn.part_ml", n_entries * nkv * nsplit * 16, 2, torch.float32,
                                        reserve=0)
        return nsplit, chunk, cluster, part_o, part_ml

    def attention_from_projection(self, ctx, qkv, k_cache, v_cache, out, block_table, q_norm_w, k_norm_w, eps,
                                  rotation, write_kv, nq, nkv, hd, page_size, scale, window=0) -> bool:
        """Decode steps: per-head norm, rotation, append to the cache and attention over the cache in one
        kernel, straight from the q/k/v projection's output.  rotation: a parts.base.Rotation or None.
        Returns False (and does nothing) when the batch, the sizes or the rotation (half-split pairs over
        the whole head) are not the ones that kernel takes; the caller then runs the steps one by one."""
        g = nq // nkv
        if (not self.fuse_decode_attention or qkv.dtype != torch.bfloat16 or ctx.max_q_len * g > 16
                or hd not in (64, 128, 256) or rotation is None or rotation.interleaved
                or 2 * rotation.pairs != hd
                or self.force_simt_attention or self.force_cp_async_decode
                or not self.lib.srlm_attention_decode_tma_takes(C.c_int(hd), C.c_int(page_size))):
            return False
        nsplit, chunk, cluster, part_o, part_ml = self._decode_plan(ctx, nkv, hd)
        self.paged_attention_decode_fused(qkv, q_norm_w, k_norm_w, eps, rotation.cos, rotation.sin, write_kv,
                                          k_cache, v_cache, out,
                                          block_table, ctx.cu_q, ctx.kv_lens, ctx.n_entries, nq, nkv, hd,
                                          page_size, scale, window, chunk, nsplit, part_o, part_ml, cluster=cluster)
        return True

    def paged_attention(self, ctx, q, k_cache, v_cache, out, block_table, nq, nkv, hd, page_size, scale,
                        window=0):
        """The product path's attention over the cache for the batch of ``ctx``: tensor cores for
        bfloat16 (keys-split when every entry is a few rows, rows-split otherwise), float32 FMA for
        the float32 path."""
        if q.dtype != torch.bfloat16 or hd % 16 or hd > 256 or self.force_simt_attention:
            self.paged_attention_simt(q, k_cache, v_cache, out, block_table, ctx.entry_of_token, ctx.positions,
                                      nq, nkv, hd, page_size, scale, window)
            return
        g = nq // nkv

        def keys_split(lo, hi):
            """Entries lo..hi-1, each of at most 16 rows (tokens x heads per KV head): the kernels that split
            the keys over blocks.  They index the step's q and out by the token offsets in cu_q, so a run of
            entries is served by handing them the run's part of cu_q, kv_lens and the block table."""
            n = hi - lo
            whole = lo == 0 and hi == ctx.n_entries
            bound = ctx.kv_bound if whole else max(ctx.host["kv_lens"][lo:hi])
            cu, kvl, table = ctx.cu_q[lo:hi + 1], ctx.kv_lens[lo:hi], block_table[lo:hi]
            if self.lib.srlm_attention_decode_tma_takes(C.c_int(hd), C.c_int(page_size)) and not self.force_cp_async_decode:
                nsplit, chunk, cluster, part_o, part_ml = self._decode_plan(ctx, nkv, hd, n, bound)
                self.paged_attention_decode_tma(q, k_cache, v_cache, out, table, cu, kvl, n, nq, nkv, hd, page_size,
                                                scale, window, chunk, nsplit, part_o, part_ml, cluster=cluster)
                return
            nsplit, chunk = self.attention_split(n, nkv, bound)
            part_o = part_ml = None
            if nsplit > 1:
                part_o = ctx.workspace.get("attn.part_o", n * nkv * nsplit * 16, hd, torch.float32, reserve=0)
                part_ml = ctx.workspace.get("attn.part_ml", n * nkv * nsplit * 16, 2, torch.float32, reserve=0)
            self.paged_attention_keys(q, k_cache, v_cache, out, table, cu, kvl, n, nq, nkv, hd, page_size, scale,
                                      window, chunk, nsplit, part_o, part_ml)

        if ctx.max_q_len * g <= 16:
            keys_split(0, ctx.n_entries)
            return
        # A mixed step: decoding requests (a row or a few) beside portions of prompts.  A row tile of the
        # rows-split kernels would be all but empty for a decoding request and would walk its keys alone,
        # one block per KV head; so the decoding requests at the head and at the tail of the batch (the
        # scheduler puts them first) go to the keys-split kernel, the rest to the rows-split one.
        q_lens = ctx.host["q_lens"]
        n = ctx.n_entries
        head = 0
        while head < n and q_lens[head] * g <= 16:
            head += 1
        tail = n
        while tail > head and q_lens[tail - 1] * g <= 16:
            tail -= 1
        # Worth a launch of its own only when the decoding requests would fill a round of blocks of the
        # rows-split kernel by themselves (one block per request and KV head) and their contexts are of
        # similar length: the two launches run one after the other, and the keys-split one lasts as long
        # as its longest request, while row tiles of all kinds share the SMs in one launch.  Measured at
        # 8B / 14B sizes: 31 decoding requests of 1,500 tokens beside a 481-token portion, 7 % / 2 % of
        # the step faster in two launches; 32 requests of 128 to 3,200 tokens, 1.5 % slower.
        short = list(range(head)) + list(range(tail, n))
        enough = self.sm_count(q.device) if self.split_mixed_min_blocks is None else self.split_mixed_min_blocks
        if self.split_mixed_attention and ctx.max_q_len > 1 and short and len(short) * nkv >= enough:
            lens = [ctx.host["kv_lens"][e] for e in short]
            if max(lens) * len(lens) > 1.5 * sum(lens):
                short = []
        else:
            short = []
        if not short:
            head, tail = 0, n
        if head > 0:
            keys_split(0, head)
        if tail < n:
            keys_split(tail, n)
        rows_entries = range(head, tail)
        def work_list(rows_per_block):
            if ctx.max_q_len == 1:
                # decode steps (more than 16 query heads per KV head): the list depends on the number of
                # entries alone, so it is made once and kept on the device; such steps are recorded into
                # CUDA graphs, and a recording must not hold a copy from a buffer that lives for one step
                lists = self.__dict__.setdefault("_decode_work_lists", {})
                key = (q.device, ctx.n_entries, g, rows_per_block)      # (every entry: head = 0, tail = n)
                if key not in lists:
                    tiles = (g + rows_per_block - 1) // rows_per_block
                    lists[key] = torch.tensor([(e, t) for e in range(ctx.n_entries) for t in range(tiles)],
                                              dtype=torch.int32).to(q.device)
                return lists[key]
            work = ctx.tables.get(("attention_rows_work", g, rows_per_block))
            if work is None:
                # the last row blocks of an entry see the most keys: they go first, so that the long
                # blocks do not start when the short ones have already left the GPU half empty
                pairs = [(e, t) for e in rows_entries
                         for t in reversed(range((q_lens[e] * g + rows_per_block - 1) // rows_per_block))]
                pairs.sort(key=lambda et: -(ctx.host["starts"][et[0]] + (et[1] + 1) * rows_per_block // g))
                work = torch.tensor(pairs, dtype=torch.int32).pin_memory().to(q.device, non_blocking=True)
                ctx.tables[("attention_rows_work", g, rows_per_block)] = work
            return work

        if (self.lib.srlm_attention_prefill_tcgen05_takes(C.c_int(hd), C.c_int(page_size))
                and not self.force_mma_sync_prefill):
            rows = [q_lens[e] * g for e in rows_entries]
            # a decode step may be replayed from a CUDA graph with longer contexts than it was recorded
            # with: its plan goes by the bound that is part of the graph's identity
            lens = [ctx.kv_bound] if ctx.max_q_len == 1 else [ctx.host["kv_lens"][e] for e in rows_entries]
            tiles, nsplit, chunk = self.prefill_attention_plan(rows, lens, nkv, self.sm_count(q.device))
            if not self.split_prefill_keys:
                nsplit, chunk = 1, 0
            work = work_list(128 * tiles)
            part_o = part_ml = None
            if nsplit > 1:
                slabs = work.shape[0] * 2 * nkv * nsplit * 128
                part_o = ctx.workspace.get("attn.rows_part_o", slabs, hd, torch.float32, reserve=0)
                part_ml = ctx.workspace.get("attn.rows_part_ml", slabs, 2, torch.float32, reserve=0)
            self.paged_attention_prefill_tcgen05(q, k_cache, v_cache, out, block_table, ctx.cu_q, ctx.kv_lens, work,
                                                 nq, nkv, hd, page_size, scale, window, tiles, nsplit, chunk, part_o,
                                                 part_ml)
            return
        tma = (hd in (64, 128) and self.lib.srlm_attention_decode_tma_takes(C.c_int(hd), C.c_int(page_size))
               and not self.force_cp_async_decode)
        if tma:
            self.paged_attention_rows_tma(q, k_cache, v_cache, out, block_table, ctx.cu_q, ctx.kv_lens,
                                          work_list(128), nq, nkv, hd, page_size, scale, window)
        else:
            self.paged_attention_rows(q, k_cache, v_cache, out, block_table, ctx.cu_q, ctx.kv_lens, work_list(64),
                                      nq, nkv, hd, page_size, scale, window)

    # ---- sampling -------------------------------------------------------------
    def argmax(self, logits, out_tokens, bad_flag):
        n, V = logits.shape
        self._check(self.lib.srlm_argmax(_ptr(logits), C.c_longlong(logits.stride(0)), C.c_int(n), C.c_int(V),
                                         _ptr(out_tokens), _ptr(bad_flag), _stream()), "argmax")

    def sample(self, logits, temperature, top_k, top_p, penalty, uniform, history, hist_offsets, out_tokens,
               bad_flag, scratch):
        """scratch: float32 [n, V] that the kernel may overwrite (the adjusted values of each row)."""
        n, V = logits.shape
        if scratch is None or scratch.dtype != torch.float32 or scratch.numel() < n * V:
            raise ShapeError("sample: scratch must hold n x V float32 values")
        self._check(self.lib.srlm_sample(_ptr(logits), C.c_longlong(logits.stride(0)), C.c_int(n), C.c_int(V),
                                         _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(penalty),
                                         _ptr(uniform), _ptr(history), _ptr(hist_offsets), _ptr(scratch),
                                         _ptr(out_tokens), _ptr(bad_flag), _stream()), "sample")


ops = KernelLibrary()
