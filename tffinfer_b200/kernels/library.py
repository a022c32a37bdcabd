"""The kernel library as the parts see it: one method per kernel, tensors in, nothing
out (outputs are arguments).  The methods check what the kernels cannot check for
themselves and pass raw device pointers to the ``extern "C"`` launchers of the
shared library built from ``csrc/``.

The reference reaches its kernels through a name-keyed callback table
("<op>_<CPU|GPU>_<dtype>", src/kernel/include/TFFOPCreatorBase.h:62-101) with a CPU
twin for some ops.  There is one backend here: sm_100a.  If the library cannot be
built or loaded, or a tensor is not on a CUDA device, the call fails loudly; nothing
falls back to another implementation.
"""
from __future__ import annotations

import ctypes
import math
import os
from typing import Optional

import numpy as np
import torch

from ..csrc import build as _build

_c_int = ctypes.c_int
_c_float = ctypes.c_float
_vp = ctypes.c_void_p

_STATUS = {
    -1: "bad argument (a size or pointer the kernel cannot take)",
    -2: "unsupported size for this kernel",
    -3: "kernel launch failed",
    -4: "CUDA driver entry point unavailable",
    -5: "a bounded wait inside a kernel ran out",
}


class KernelError(RuntimeError):
    pass


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {t.dtype}")


def _ptr(t: Optional[torch.Tensor]):
    return _vp(t.data_ptr()) if t is not None else _vp(0)


def effective_requests(kv_lens) -> float:
    """sum(context) / max(context): how many requests of the longest context read as many keys as these
    do.  A step's decoded tokens are one (request, key/value head) work item each unless the key range is
    shared out; the longest context sets how long the longest item runs, the sum how long all of them
    take together, so this ratio, not the number of requests, says how many shares the key range needs."""
    kv = np.asarray(kv_lens, dtype=np.float64)
    if kv.size == 0 or kv.max() <= 0:
        return 1.0
    return float(kv.sum() / kv.max())


def nearest_power_of_two(x: float) -> int:
    b = 1
    while b * 1.4142 < x:
        b *= 2
    return b


class DeferredNorm:
    """A norm that has not been run yet: the float32 rows ``x``, the weight and eps of an RMSNorm whose
    output only feeds a product of the kernel library.  ``CudaKernels.gated_mlp`` takes it in place of the
    activation rows and runs norm, product and SwiGLU as one kernel when the shape allows (decode steps of at
    most 16 tokens in bfloat16: csrc/gemm_tc_cluster.cu); otherwise, and in ``qkv_project``, the norm kernel
    runs first (``materialize``)."""
    def __init__(self, x, weight, eps, out_dtype, ops):
        self.x, self.weight, self.eps, self.out_dtype, self.ops = x, weight, float(eps), out_dtype, ops
        self.shape = x.shape
        self.dtype = out_dtype
        self.device = x.device

    def materialize(self):
        out = torch.empty(self.x.shape, dtype=self.out_dtype, device=self.x.device)
        self.ops.rmsnorm(self.x, self.weight, self.eps, out)
        return out


class CudaKernels:
    """Loads (building first if needed) the sm_100a kernel library."""

    def __init__(self, verbose_build: bool = True):
        if not torch.cuda.is_available():
            raise KernelError("tffinfer_b200 needs a CUDA device (sm_100a): torch.cuda.is_available() is False")
        path = _build.library_path(build=True, verbose=verbose_build)
        try:
            self.lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError(f"cannot load the kernel library {path}: {e}") from None
        self.path = path
        self.launches = 0          # number of kernel launches issued through this object
        self._accumulators = {}    # (shape, device) -> float32 buffer kept at zero between uses
        self._acc_zero = {}        # data_ptr -> True while the buffer is known to hold zeros
        self._inv_freq_cache = {}
        self._moe_counts = {}      # (experts, device) -> int32 counters that the routed feed-forward keeps at zero
        # the planners below cut work by the SM count the launchers size their grids with
        self.NUM_SMS = int(self.lib.tff_sm_count())
        if self.NUM_SMS <= 0:
            raise KernelError("cannot read the SM count of the current CUDA device")

    # ------------------------------------------------------------- plumbing
    @staticmethod
    def _stream():
        return _vp(torch.cuda.current_stream().cuda_stream)

    def _check(self, status: int, what: str) -> None:
        if status != 0:
            raise KernelError(f"{what}: {_STATUS.get(status, f'status {status}')}")

    @staticmethod
    def _need_cuda(*tensors) -> None:
        for t in tensors:
            if t is not None and not t.is_cuda:
                raise KernelError("a tensor given to a CUDA kernel is not on a CUDA device")
            if t is not None and not t.is_contiguous():
                raise KernelError("kernels take contiguous tensors")

    @staticmethod
    def _cache_args(kv_cache, kv_layer: int):
        """(pointer, pages, layers, layer) of a paged cache [pages, layers, 2, kv heads, page, head] as the
        launchers take them.  The tensor is either contiguous as it reads (pages outermost), or that shape
        as a view of storage with the layers outermost, each layer's pages then lying together (what the
        engine allocates: a layer's attention reads addresses within one layer's share of the pool and not
        64 KB out of every ``layers`` x 64 KB).  For the second the launcher is given the layer's own
        [pages, 1, ...] block."""
        if kv_cache is None:
            return _vp(0), 0, 1, kv_layer
        if not kv_cache.is_cuda:
            raise KernelError("a tensor given to a CUDA kernel is not on a CUDA device")
        if kv_cache.is_contiguous():
            return _vp(kv_cache.data_ptr()), kv_cache.shape[0], kv_cache.shape[1], kv_layer
        st, block = kv_cache.stride(), 1
        for i in range(kv_cache.dim() - 1, 1, -1):             # the [2, kv heads, page, head] block of a page is dense
            if st[i] != block:
                break
            block *= kv_cache.shape[i]
        else:
            if st[0] == block and st[1] == block * kv_cache.shape[0]:
                return (_vp(kv_cache.data_ptr() + kv_layer * st[1] * kv_cache.element_size()),
                        kv_cache.shape[0], 1, 0)
        raise KernelError("the cache is neither contiguous nor a view of layer-major storage")

    # -------------------------------------------------------------- kernels
    def embed(self, token_ids, table, out, scale: float = 1.0, copies: int = 0) -> None:
        """out[t] = table[token_ids[t]] * scale; with ``copies`` = S > 0, out is [T, S, H] and every copy gets it."""
        self._need_cuda(token_ids, table, out)
        if copies > 0:
            T, S, H = out.shape
            assert S == copies and token_ids.dtype == torch.int32 and out.dtype == torch.float32 and table.shape[1] == H
            self._check(self.lib.tff_embed_streams(_ptr(token_ids), _ptr(table), _c_int(_dt(table)), _ptr(out), _c_int(T),
                                                   _c_int(H), _c_int(table.shape[0]), _c_float(scale), _c_int(S),
                                                   self._stream()), "embed_streams")
            self.launches += 1
            return
        T, H = out.shape
        assert token_ids.dtype == torch.int32 and out.dtype == torch.float32 and table.shape[1] == H
        self._check(self.lib.tff_embed(_ptr(token_ids), _ptr(table), _c_int(_dt(table)), _ptr(out),
                                       _c_int(T), _c_int(H), _c_int(table.shape[0]), _c_float(scale), self._stream()), "embed")
        self.launches += 1

    def logit_transform(self, logits, scale: float = 1.0, softcap: float = 0.0) -> None:
        """In place: logits * scale, then softcap * tanh(. / softcap) when softcap > 0."""
        self._need_cuda(logits)
        assert logits.dtype == torch.float32
        self._check(self.lib.tff_logit_transform(_ptr(logits), ctypes.c_longlong(logits.numel()), _c_float(scale),
                                                 _c_float(softcap), self._stream()), "logit_transform")
        self.launches += 1

    def rmsnorm(self, x, weight, eps: float, out, row_index=None) -> None:
        self._need_cuda(x, weight, out, row_index)
        rows, dim = out.shape
        assert x.dtype == torch.float32 and weight.dtype == torch.float32 and x.shape[1] == dim
        assert weight.numel() == dim
        if row_index is not None:
            assert row_index.dtype == torch.int32 and row_index.numel() == rows
        else:
            assert x.shape[0] == rows
        self._check(self.lib.tff_rmsnorm(_ptr(x), _ptr(weight), _ptr(row_index), _ptr(out), _c_int(_dt(out)),
                                         _c_int(rows), _c_int(dim), _c_float(eps), self._stream()), "rmsnorm")
        self.launches += 1

    def rmsnorm_pair(self, x, weight_a, weight_b, eps: float, out_a, out_b) -> None:
        """Two RMS norms of the same float32 rows with a weight each, the rows read once (a layer whose two sublayers
        each norm the same residual)."""
        self._need_cuda(x, weight_a, weight_b, out_a, out_b)
        rows, dim = x.shape
        assert x.dtype == weight_a.dtype == weight_b.dtype == torch.float32 and weight_a.numel() == weight_b.numel() == dim
        assert out_a.dtype == out_b.dtype and tuple(out_a.shape) == tuple(out_b.shape) == (rows, dim)
        self._check(self.lib.tff_rmsnorm_pair(_ptr(x), _ptr(weight_a), _ptr(weight_b), _ptr(out_a), _ptr(out_b),
                                              _c_int(_dt(out_a)), _c_int(rows), _c_int(dim), _c_float(eps), self._stream()),
                    "rmsnorm_pair")
        self.launches += 1

    def gemm(self, a, w, out, residual=None) -> None:
        """out[M, N] = a[M, K] @ w[N, K]^T (+ residual, float32 [M, N]; may be ``out``)."""
        self._need_cuda(a, w, out, residual)
        M, K = a.shape
        N = w.shape[0]
        assert w.shape[1] == K and tuple(out.shape) == (M, N)
        if residual is not None:
            assert residual.dtype == torch.float32 and tuple(residual.shape) == (M, N)
            assert out.dtype == torch.float32
        self._gemm_dispatch(a, w, out, residual, M, N, K)

    def _gemm_dispatch(self, a, w, out, residual, M, N, K) -> None:
        if (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and K % 8 == 0
                and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0):
            self.gemm_tc(a, w, out, residual)
        else:
            self.gemm_simt(a, w, out, residual)

    def gemm_simt(self, a, w, out, residual=None) -> None:
        """Plain-FMA float32-accumulate product for any mix of float32 / bfloat16 operands."""
        M, K = a.shape
        N = w.shape[0]
        self._check(self.lib.tff_gemm_simt(_ptr(a), _c_int(_dt(a)), _ptr(w), _c_int(_dt(w)), _ptr(out),
                                           _c_int(_dt(out)), _ptr(residual), _c_int(M), _c_int(N), _c_int(K),
                                           self._stream()), "gemm_simt")
        if out.data_ptr() in self._acc_zero:
            self._acc_zero[out.data_ptr()] = False     # an accumulator buffer that now holds a product
        self.launches += 1

    FOLD_MAX_M = 16           # up to this many rows the norm is folded into the gate/up product (with SwiGLU)
    CLUSTER_MAX_M = 16        # up to this many rows the gate/up product applies SwiGLU itself (clusters share a tile's K range)
    FOLD_DECODE = os.environ.get("TFFINFER_FOLD_DECODE", "1") != "0"
    SWAP_MAX_M = 256          # up to this many rows the weights are the 128-row operand
    USE_SM_PAIRS = os.environ.get("TFFINFER_SM_PAIRS", "1") != "0"   # prompt-sized products on tcgen05 cta_group::2
    NUM_SMS = 0               # SMs of the device, read from it when the library is loaded

    def tc_plan(self, M: int, N: int, K: int, out_is_f32: bool, add: bool = False):
        """(swap, bn, stream_k) of the tcgen05 product for a shape.  stream_k: 0 = whole tiles; 1 = the
        (tile, K block) units in equal contiguous shares; S >= 2 = the tiles of the last, partial wave
        in S slices of their K range."""
        if M <= self.SWAP_MAX_M:
            bn = 16
            while bn < M:
                bn *= 2
            tiles = -(-N // 128)
            stream_k = 1 if (out_is_f32 and tiles < 4 * self.NUM_SMS) else 0
            return 1, bn, stream_k
        return self.prompt_plan(M, N, K, add and out_is_f32)

    # What a wave of tiles costs in each of the three prompt-sized configurations, in us per K block of 64 at the
    # clocks of a B200 under load, and what a launch costs on top: fitted to the measured times of the q/k/v, o,
    # gate/up and down products of the 8B and 14B shapes at 160 to 544 rows (within 10 %; only the ratios matter).
    # A tile of the last wave costs as much as one of a full wave, so the plan with the fewest waves wins unless
    # its tiles are the dearer ones: 544 rows of the 14B shape's q/k/v are 84 pair tiles on 74 pairs of SMs (two
    # waves, 63 us) and 140 single tiles on 148 SMs (one wave, 38 us).
    #          bn: (us a K block and wave, us a launch, tile rows, tile columns, SMs a tile)
    TILE_COST = {512: (0.385, 3.0, 256, 256, 2), 256: (0.450, 1.0, 128, 256, 1), 128: (0.340, 1.5, 128, 128, 1)}

    def prompt_costs(self, M: int, N: int, K: int, added: bool, kinds=(512, 256, 128)):
        """{bn: (estimated us, slices)} of the normal-orientation configurations for a prompt-sized product; the
        last wave's tiles are cut along K only where the result is added to a float32 buffer."""
        kb = -(-K // 64)
        costs = {}
        for bn in kinds:
            if bn == 512 and (not self.USE_SM_PAIRS or N <= 128):
                continue
            c, launch, tm, tn, sms = self.TILE_COST[bn]
            tiles, slots = -(-M // tm) * -(-N // tn), max(1, self.NUM_SMS // sms)
            waves, tail = divmod(tiles, slots)
            slices = self.tail_slices(tiles, kb, slots) if added else 0
            if tail:
                waves += (-(-tail * slices // slots) / slices + 0.02 * slices) if slices else 1
            costs[bn] = (waves * kb * c + launch, slices)
        return costs

    def prompt_plan(self, M: int, N: int, K: int, added: bool, kinds=(512, 256, 128)):
        """(0, bn, slices) of the cheapest of them."""
        costs = self.prompt_costs(M, N, K, added, kinds)
        bn = min(costs, key=lambda b: costs[b][0])
        return 0, bn, costs[bn][1]

    @staticmethod
    def tail_slices(tiles: int, k_blocks: int, ctas: int) -> int:
        """In how many slices the K range of the tiles of the last wave is cut (0: not at all).  A wave of
        R tiles in S slices takes ceil(R*S/G)/S of a tile's time; every slice costs another pass of the
        tile through the epilogue, here put at 2 % of a tile's time."""
        tail = tiles % ctas
        if tail == 0:
            return 0
        best, best_cost = 0, 1.0
        for s in range(2, min(8, k_blocks) + 1):
            cost = -(-tail * s // ctas) / s + 0.02 * s
            if cost < best_cost - 1e-9:
                best, best_cost = s, cost
        return best

    def gemm_tc(self, a, w, out, residual=None, plan=None) -> None:
        """bfloat16 x bfloat16 product on the tensor cores (tcgen05), float32 accumulation."""
        M, K = a.shape
        N = w.shape[0]
        swap, bn, stream_k = plan if plan is not None else self.tc_plan(M, N, K, out.dtype == torch.float32,
                                                                        residual is not None)
        add = 0
        if residual is not None:
            assert out.dtype == torch.float32
            if residual.data_ptr() != out.data_ptr():
                out.copy_(residual)
            add = 1
        elif stream_k:
            assert out.dtype == torch.float32
            if not self._acc_zero.get(out.data_ptr(), False):
                self.zero_f32(out)            # shares of a split tile are added to it
        if out.data_ptr() in self._acc_zero:
            self._acc_zero[out.data_ptr()] = False
        self._check(self.lib.tff_gemm_tc(_ptr(a), _ptr(w), _ptr(out), _c_int(_dt(out)), _c_int(add),
                                         _c_int(M), _c_int(N), _c_int(K), _c_int(swap), _c_int(bn), _c_int(stream_k),
                                         self._stream()), "gemm_tc")
        self.launches += 1

    def zero_f32(self, t) -> None:
        assert t.dtype == torch.float32 and t.is_contiguous()
        self._check(self.lib.tff_zero_f32(_ptr(t), ctypes.c_longlong(t.numel()), self._stream()), "zero_f32")
        self.launches += 1

    def reset_state_slots(self, state, slots, pos_start) -> None:
        """state[slots[b]] = 0 for every request b of the step whose first token is at position 0.
        state: [slots, ...] of any element type; slots, pos_start: int32 [B] on the device."""
        self._need_cuda(state, slots, pos_start)
        assert slots.dtype == pos_start.dtype == torch.int32 and slots.numel() == pos_start.numel()
        slot_bytes = state[0].numel() * state.element_size()
        self._check(self.lib.tff_reset_state_slots(_ptr(state), ctypes.c_longlong(slot_bytes), _c_int(state.shape[0]),
                                                   _ptr(slots), _ptr(pos_start), _c_int(slots.numel()),
                                                   self._stream()), "reset_state_slots")
        self.launches += 1

    def gather_tokens(self, token_ids, drawn, src) -> None:
        """token_ids[i] = drawn[src[i]] wherever src[i] >= 0 (all int32, on the device)."""
        self._need_cuda(token_ids, drawn, src)
        assert token_ids.dtype == drawn.dtype == src.dtype == torch.int32 and src.numel() == token_ids.numel()
        self._check(self.lib.tff_gather_tokens(_ptr(token_ids), _ptr(drawn), _ptr(src), _c_int(token_ids.numel()),
                                               _c_int(drawn.numel()), self._stream()), "gather_tokens")
        self.launches += 1

    def error_word_async(self, pinned: torch.Tensor, index: int) -> None:
        """Copies the kernels' error word into element ``index`` of a pinned int32 host tensor, in stream
        order; non-zero there (once the stream has got that far) means check_errors() will raise."""
        assert pinned.dtype == torch.int32 and pinned.is_pinned() and 0 <= index < pinned.numel()
        self._check(self.lib.tff_error_word_to_host_async(_vp(pinned.data_ptr() + 4 * index), self._stream()),
                    "error_word_to_host")

    def selftest_bounded_wait(self, arrive: bool, max_polls: int = 4096) -> None:
        """Launches a kernel that waits, bounded, on a barrier at which one thread arrives (``arrive``) or
        nobody does: in the second case the wait runs out after ``max_polls`` polls and raises the error
        word, as a stalled pipeline inside a tcgen05 kernel would.  For testing the way from the word to
        the caller (error_word_async, check_errors)."""
        self._check(self.lib.tff_selftest_bounded_wait(_c_int(1 if arrive else 0), _c_int(max_polls), self._stream()),
                    "selftest_bounded_wait")
        self.launches += 1

    def check_errors(self) -> None:
        """Synchronises and raises if a bounded wait inside a kernel ran out since the last check."""
        v = self.lib.tff_kernel_error()
        if v != 0:
            raise KernelError("a bounded wait inside a tcgen05 kernel ran out (or the error word could not be read)")

    @staticmethod
    def gate_up_block(inter: int) -> int:
        """Layout of a merged gate/up weight: 64 = gate and up rows alternate in blocks of 64 (what the
        fused tensor-core epilogue wants), 0 = all gate rows, then all up rows."""
        return 64 if inter % 64 == 0 else 0

    def merge_gate_up(self, gate_w, up_w):
        """One weight [2I, K] from the gate and up projections, in the layout gemm_swiglu expects."""
        I, K = gate_w.shape
        b = self.gate_up_block(I)
        if b == 0:
            return torch.cat([gate_w, up_w], dim=0).contiguous()
        return torch.stack([gate_w.view(I // b, b, K), up_w.view(I // b, b, K)], dim=1).reshape(2 * I, K).contiguous()

    # ------------------------------------------------------- accumulator buffers
    def projection_buffer(self, rows: int, width: int, device, act_dtype, use: str = "") -> torch.Tensor:
        """A float32 [rows, width] buffer for a projection's accumulators.  For decode-sized bfloat16
        batches it is a persistent buffer that is zero now and that its reader sets back to zero
        (``release_input`` of qk_norm_rope_kv_write, ``clear`` of swiglu), so that the split product
        can add into it without a clearing kernel; otherwise it is plain scratch.  Buffers of different ``use`` are
        different buffers: a product that runs while a sublayer's output of the same shape is still waiting for its
        reader names a use of its own."""
        if act_dtype != torch.bfloat16 or rows > self.SWAP_MAX_M:
            return torch.empty((rows, width), dtype=torch.float32, device=device)
        key = (rows, width, str(device), use)
        buf = self._accumulators.get(key)
        if buf is None:
            buf = torch.zeros((rows, width), dtype=torch.float32, device=device)
            self._accumulators[key] = buf
            self._acc_zero[buf.data_ptr()] = True
        return buf

    def sublayer_output(self, rows: int, width: int, device, act_dtype) -> torch.Tensor:
        """A float32 [rows, width] buffer for a sublayer's output that a connector consumes (``stream_step`` clears it
        behind the read): for decode-sized bfloat16 steps one of the accumulator buffers, so that the split product
        that writes it needs no clearing kernel; else plain scratch."""
        return self.projection_buffer(rows, width, device, act_dtype)

    def reset_accumulators(self) -> None:
        """After a step that was cut short: every accumulator buffer back to zero."""
        for buf in self._accumulators.values():
            buf.zero_()
            self._acc_zero[buf.data_ptr()] = True
        for counts in self._moe_counts.values():
            counts.zero_()

    # ------------------------------------------------------- folded decode products
    def can_fold_norm(self, x, weight, out_dtype) -> bool:
        """Whether an RMSNorm of these rows may be handed to the products as a DeferredNorm."""
        return (self.FOLD_DECODE and x.is_cuda and out_dtype == torch.bfloat16 and x.dtype == torch.float32
                and x.dim() == 2 and x.shape[0] <= self.FOLD_MAX_M and x.shape[1] % 8 == 0 and x.is_contiguous()
                and weight.dtype == torch.float32 and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)

    def _foldable_weight(self, w) -> bool:
        return w.dtype == torch.bfloat16 and w.is_contiguous() and w.data_ptr() % 16 == 0 and w.shape[1] % 8 == 0

    ACTIVATION_CODES = {"silu": 0, "gelu_tanh": 1, "relu2": 2}    # relu2: the square of relu, of one product (not gated)

    def gated_mlp(self, h, w_gate_up, w_down, residual, inter: int, activation: str = "silu", out=None) -> None:
        """residual += down(act(gate(h)) * up(h)); ``h`` the activation rows or a DeferredNorm of them.  With
        ``residual`` None the result goes to ``out`` (float32 [T, hidden]) instead.  ``activation``: "silu" or
        "gelu_tanh" (the tanh form of gelu).
        A decode step of at most FOLD_MAX_M tokens in bfloat16 whose norm has been deferred runs two kernels:
        norm, gate/up product and activation as one (clusters of CTAs share a tile's K range), then the down
        product.  Everything else runs the products and kernels one by one."""
        T = h.shape[0]
        code = self.ACTIVATION_CODES[activation]
        target = residual if residual is not None else out

        def down(act):
            if residual is None:
                self.gemm(act, w_down, out)
            else:
                self.gemm(act, w_down, residual, residual=residual)

        if isinstance(h, DeferredNorm):
            if (self.gate_up_block(inter) == 64 and self._foldable_weight(w_gate_up)
                    and target.is_cuda and target.dtype == torch.float32):
                act = torch.empty((T, inter), dtype=torch.bfloat16, device=target.device)
                self._need_cuda(h.x, h.weight, w_gate_up, act)
                assert tuple(w_gate_up.shape) == (2 * inter, h.x.shape[1])
                self._check(self.lib.tff_gemm_tc_cluster_gated(
                    _ptr(h.x), _ptr(h.weight), _c_float(h.eps), _ptr(w_gate_up), _c_int(T), _c_int(h.x.shape[1]),
                    _ptr(act), _c_int(inter), _c_int(code), self._stream()), "gemm_tc_cluster_gated")
                self.launches += 1
                down(act)
                return
            h = h.materialize()
        act = torch.empty((T, inter), dtype=h.dtype, device=h.device)
        if (self.FOLD_DECODE and T <= self.CLUSTER_MAX_M and h.dtype == torch.bfloat16 and h.is_cuda and h.is_contiguous()
                and self.gate_up_block(inter) == 64 and self._foldable_weight(w_gate_up) and h.data_ptr() % 16 == 0):
            # the product with the activation in the first CTA of each cluster: no float32 accumulators, no activation kernel
            self._need_cuda(h, w_gate_up, act)
            assert tuple(w_gate_up.shape) == (2 * inter, h.shape[1])
            self._check(self.lib.tff_gemm_tc_cluster_gated_bf16(_ptr(h), _ptr(w_gate_up), _c_int(T), _c_int(h.shape[1]),
                                                                _ptr(act), _c_int(inter), _c_int(code), self._stream()),
                        "gemm_tc_cluster_gated_bf16")
            self.launches += 1
        else:
            self.gemm_gated_act(h, w_gate_up, act, activation)
        down(act)

    def swiglu(self, gate_up, out, block: int = 0) -> None:
        """out[t, i] = silu(gate[t, i]) * up[t, i]; gate_up float32 or of out's type, [gate | up] (block = 0) or
        alternating in blocks of ``block`` columns."""
        self._need_cuda(gate_up, out)
        T, I = out.shape
        assert gate_up.shape == (T, 2 * I) and gate_up.dtype in (torch.float32, out.dtype)
        clear = 1 if gate_up.data_ptr() in self._acc_zero else 0
        self._check(self.lib.tff_swiglu(_ptr(gate_up), _c_int(_dt(gate_up)), _ptr(out), _c_int(_dt(out)),
                                        _c_int(T), _c_int(I), _c_int(block), _c_int(clear), self._stream()), "swiglu")
        if clear:
            self._acc_zero[gate_up.data_ptr()] = True
        self.launches += 1

    def gated_act(self, gate_up, out, block: int = 0, activation: str = "silu") -> None:
        """out[t, i] = act(gate[t, i]) * up[t, i], the layouts of ``swiglu``; act "silu" or "gelu_tanh"."""
        self._need_cuda(gate_up, out)
        T, I = out.shape
        assert gate_up.shape == (T, 2 * I) and gate_up.dtype in (torch.float32, out.dtype)
        clear = 1 if gate_up.data_ptr() in self._acc_zero else 0
        self._check(self.lib.tff_gated_act(_ptr(gate_up), _c_int(_dt(gate_up)), _ptr(out), _c_int(_dt(out)), _c_int(T),
                                           _c_int(I), _c_int(block), _c_int(clear),
                                           _c_int(self.ACTIVATION_CODES[activation]), self._stream()), "gated_act")
        if clear:
            self._acc_zero[gate_up.data_ptr()] = True
        self.launches += 1

    # ------------------------------------------------------- residual of several streams
    def stream_step(self, x, y=None, scale=None, mix=None, out=None, read=None, norm_weight=None, eps: float = 0.0,
                    h=None, row_index=None, total=None, bias=None) -> None:
        """x float32 [T, S, W], the residual's streams.  With ``y`` (float32 [T, W]): x_t <- sum_s mix[s, t] x_s +
        out[t] * (scale * y) in place (mix [S, S], out [S], scale [W]; None = identity, ones, ones).  With ``h``
        ([rows, W], activation type): h = rmsnorm(sum_s read[s] x_s) with ``norm_weight`` and ``eps`` (read None = ones).
        With ``total`` (float32 [rows, W]): the combined row itself.  ``row_index`` (int32 [rows]) limits all of it to
        those rows of x; h and total are then indexed by the place in ``row_index``, and x itself is left as it was
        (the new streams of those rows feed h only).  ``bias`` (float32 [W]): added to every stream behind the write and
        ahead of the read."""
        self._need_cuda(x, y, scale, mix, out, read, norm_weight, h, row_index, total, bias)
        assert bias is None or (bias.dtype == torch.float32 and bias.numel() == x.shape[2])
        T, S, W = x.shape
        assert x.dtype == torch.float32
        for t in (y, scale, mix, out, read, norm_weight, total):
            assert t is None or t.dtype == torch.float32
        assert y is None or tuple(y.shape) == (T, W)
        assert mix is None or mix.numel() == S * S
        assert out is None or out.numel() == S
        assert read is None or read.numel() == S
        assert scale is None or scale.numel() == W
        rows = T if row_index is None else row_index.numel()
        if row_index is not None:
            assert row_index.dtype == torch.int32
        if h is not None:
            assert tuple(h.shape) == (rows, W)
        if total is not None:
            assert tuple(total.shape) == (rows, W)
        # a y that is one of the accumulator buffers kept at zero is cleared behind the read; when only some rows are
        # read (row_index; a row may be listed twice), nothing is cleared and the buffer counts as used
        kept_zero = y is not None and y.data_ptr() in self._acc_zero
        clear = 1 if (kept_zero and row_index is None) else 0
        self._check(self.lib.tff_stream_step(_ptr(x), _c_int(S), _c_int(W), _ptr(y), _c_int(clear), _ptr(scale), _ptr(mix), _ptr(out),
                                             _ptr(read), _ptr(norm_weight), _c_float(eps), _ptr(row_index), _ptr(h),
                                             _c_int(_dt(h)) if h is not None else _c_int(0), _ptr(total), _c_int(rows),
                                             _ptr(bias), self._stream()), "stream_step")
        if kept_zero:
            self._acc_zero[y.data_ptr()] = bool(clear)
        self.launches += 1

    # ------------------------------------------------------- mixers with a rotation computed on the fly
    def qkv_finish(self, proj, q_out, k_out, freq, batch, block_table, kv_cache, kv_layer, page_size, nq, nkv, d, dv,
                   k_scale: float = 1.0, v_mode: int = 0, v_share=None, lam=None, gate_off: int = -1, gate_out=None,
                   last_reader: bool = True, proj_off: int = 0, bias=None, unit_eps: float = 0.0) -> None:
        """proj [T, ld] = [q (nq*d) | k (nkv*d) | v (nkv*dv) | ...] -> rotated q in ``q_out`` [T, nq*d]; rotated k
        (times ``k_scale``) and v into the tokens' cache slots or, with no cache, k into ``k_out`` (float32);
        ``freq`` = (frequencies, rot_dim, magnitude, interleaved) or None; value mixing and head gates as
        csrc/qkv_finish.cu describes them.  When ``proj`` is one of the accumulator buffers that are kept at zero
        between uses, what the kernel consumes is set back to zero; ``last_reader`` says that nothing of the row is
        left for another kernel (which then clears the rest).  ``proj_off``: the row's q starts at that column.
        ``bias``: float32 [nq*d + nkv*d + nkv*dv] added to q, k and v first; ``unit_eps`` > 0: every q and k head is
        divided by sqrt(mean(x^2) + unit_eps) behind the rotation (an RMS norm without a weight)."""
        self._need_cuda(proj, q_out, k_out, block_table, v_share, lam, gate_out, bias)
        assert bias is None or (bias.dtype == torch.float32 and bias.numel() == nq * d + nkv * d + nkv * dv)
        T, ld = proj.shape
        f, rot, mag, inter = freq if freq is not None else (None, 0, 1.0, False)
        c_ptr, _, c_layers, c_layer = self._cache_args(kv_cache, kv_layer)
        dc = kv_cache.shape[-1] if kv_cache is not None else 0
        if kv_cache is not None:
            assert tuple(kv_cache.shape[2:5]) == (2, nkv, page_size)
        clear = 1 if proj.data_ptr() in self._acc_zero else 0
        self._check(self.lib.tff_qkv_finish(
            _vp(proj.data_ptr() + proj_off * proj.element_size()), _c_int(_dt(proj)), _c_int(clear), _c_int(ld), _ptr(q_out),
            _c_int(_dt(q_out)), _ptr(k_out),
            _ptr(f), _c_int(rot), _c_float(mag), _c_int(1 if inter else 0), _c_float(k_scale),
            _ptr(batch.positions), _ptr(batch.tok_req), _ptr(block_table),
            _c_int(block_table.shape[1] if block_table is not None else 0),
            c_ptr, _c_int(_dt(kv_cache)) if kv_cache is not None else _c_int(0), _c_int(c_layers), _c_int(c_layer),
            _c_int(page_size), _c_int(dc), _c_int(v_mode), _ptr(v_share), _ptr(lam), _c_int(gate_off), _ptr(gate_out),
            _c_int(T), _c_int(nq), _c_int(nkv), _c_int(d), _c_int(dv), _ptr(bias), _c_float(unit_eps), self._stream()),
            "qkv_finish")
        if clear and last_reader:
            self._acc_zero[proj.data_ptr()] = True
        self.launches += 1

    def attend_gated(self, h, w_in, freq, batch, block_table, kv_cache, kv_layer, page_size, out, nq, nkv, d, dv,
                     scale, window, softcap, sink, v_mode, v_share, lam, gate_off, write_cache, pre=None) -> None:
        """The whole of a gated, capped, sink attention between its input rows and its output projection: one product
        for q, k, v and the head gates (``w_in`` rows [q | k | v | gates | padding]); rotation, value mixing, cache
        write and sigmoid of the gates; attention over the paged cache with the cap, the window, the sink and the
        gates -> out [T, nq*dv].  ``pre`` = dict(taps, conv=(q, k, v weights [channels, taps] or None), norm=(q, k weights
        over the whole projection or None), eps, state): a short causal convolution over time on the projected q, k, v
        and an RMS norm of all of q and of all of k, between the product and the rotation (short_conv_norm)."""
        if not write_cache:
            raise KernelError("attend_gated writes the keys and values it attends to; a borrowed cache is not supported")
        T = h.shape[0]
        if isinstance(h, DeferredNorm):
            h = h.materialize()
        proj = self.projection_buffer(T, w_in.shape[0], h.device, h.dtype)
        self.gemm(h, w_in, proj)
        q = torch.empty((T, nq * d), dtype=out.dtype, device=out.device)
        gates = torch.empty((T, nq), dtype=torch.float32, device=out.device) if gate_off >= 0 else None
        if pre is not None:
            taps = int(pre.get("taps") or 1)
            conv = pre.get("conv") or (None, None, None)
            norm = pre.get("norm") or (None, None)
            widths = (nq * d, nkv * d, nkv * dv)
            if v_mode == 0 and self.CONV_FINISH and (sum(widths) + widths[0] + widths[1] + 32 + d) * 4 <= 200 * 1024:
                # convolution, norms, rotation, cache write and gates in one pass over the accumulators
                conv_t = pre.get("conv_t") or tuple(w.t().contiguous() if w is not None else None for w in conv)
                self.conv_finish(proj, conv_t, norm, taps, float(pre.get("eps", 0.0)), pre.get("state"), q, freq, batch,
                                 block_table, kv_cache, kv_layer, page_size, nq, nkv, d, dv, gate_off, gates)
                self.short_conv_state(proj, taps, sum(widths), pre.get("state"), batch)
                self.attention_ext(q, batch, block_table, kv_cache, kv_layer, page_size, out, nq, nkv, d, dv, scale,
                                   window, softcap, sink, gates)
                return
            mixed = torch.empty((T, proj.shape[1]), dtype=torch.float32, device=proj.device)
            self.short_conv_norm(proj, mixed, [(widths[0], conv[0], norm[0]), (widths[1], conv[1], norm[1]),
                                               (widths[2], conv[2], None)], taps, float(pre.get("eps", 0.0)),
                                 pre.get("state"), batch)
            self.short_conv_state(proj, taps, sum(widths), pre.get("state"), batch)
            proj = mixed
        self.qkv_finish(proj, q, None, freq, batch, block_table, kv_cache, kv_layer, page_size, nq, nkv, d, dv,
                        1.0, v_mode, v_share, lam, gate_off, gates)
        self.attention_ext(q, batch, block_table, kv_cache, kv_layer, page_size, out, nq, nkv, d, dv, scale, window,
                           softcap, sink, gates)

    @staticmethod
    def _sink_args(sink, nq: int):
        """(on, per-head scores or None) of a softmax sink given as False, True (score 0) or a float32 tensor [nq]."""
        if isinstance(sink, torch.Tensor):
            if sink.dtype != torch.float32 or sink.numel() != nq or not sink.is_cuda or not sink.is_contiguous():
                raise KernelError("a sink's scores are a contiguous float32 tensor [heads] on the device")
            return True, sink
        return bool(sink), None

    def attention_ext(self, q, batch, block_table, kv_cache, kv_layer, page_size, out, nq, nkv, d, dv, scale, window,
                      softcap: float = 0.0, sink=False, gates=None) -> None:
        """q [T, nq*d] against the paged cache (slots of kv_cache.shape[-1] >= max(d, dv) elements) -> out [T, nq*dv],
        with a cap on the scores, a sink in the softmax (True: of score 0; a float32 tensor [nq]: of that score per head)
        and a multiplier per (token, head)."""
        self._need_cuda(q, block_table, out, gates)
        T = q.shape[0]
        dc = kv_cache.shape[-1]
        assert kv_cache.dtype == q.dtype == out.dtype
        assert tuple(q.shape) == (T, nq * d) and tuple(out.shape) == (T, nq * dv)
        assert tuple(kv_cache.shape[2:]) == (2, nkv, page_size, dc) and dc >= max(d, dv)
        assert gates is None or (gates.dtype == torch.float32 and tuple(gates.shape) == (T, nq))
        if q.dtype == torch.bfloat16 and d == dv == dc and d in (64, 128) and hasattr(batch, "h_sorted_q_lens"):
            # the kernels of plain attention take the cap, the sink and the gates as well
            self.attention_bf16(q, batch, block_table, kv_cache, kv_layer, page_size, out, nq, nkv, d, scale, window,
                                extra=(float(softcap), sink, gates))
            return
        c_ptr, _, c_layers, c_layer = self._cache_args(kv_cache, kv_layer)
        sink_on, sink_val = self._sink_args(sink, nq)
        self._check(self.lib.tff_attention_generic_ext(
            _ptr(q), _c_int(_dt(q)), _c_int(q.shape[1]),
            _ptr(batch.positions), _ptr(batch.tok_req), _ptr(block_table), _c_int(block_table.shape[1]),
            c_ptr, _c_int(c_layers), _c_int(c_layer), _c_int(page_size),
            _ptr(out), _c_int(T), _c_int(nq), _c_int(nkv), _c_int(d), _c_int(dv), _c_int(dc), _c_float(scale),
            _c_int(window), _c_float(softcap), _c_int(1 if sink_on else 0), _ptr(sink_val), _ptr(gates), self._stream()),
            "attention_generic_ext")
        self.launches += 1

    def retain(self, h, w_in, freq, batch, state, decay, out, H, d, dv, k_scale: float, eps: float) -> None:
        """The whole of a retention mixer between its input rows and its output projection: one product for q, k, v
        and the gate (``w_in`` rows [q | k | v | gate | padding]) into float32; rotation of q and k (k times
        ``k_scale``), float32; the recurrence over ``state`` [slots, H, d, dv] with ``decay`` [H], the per-head RMS
        norm and the silu gate -> out [T, H*dv].  Steps in which every request brings one token run token by token,
        the others chunk by chunk."""
        T = h.shape[0]
        if isinstance(h, DeferredNorm):
            h = h.materialize()
        self._need_cuda(state, decay, out)
        assert state.dtype == torch.float32 and tuple(state.shape[1:]) == (H, d, dv) and decay.numel() == H
        proj = self.projection_buffer(T, w_in.shape[0], h.device, h.dtype)
        self.gemm(h, w_in, proj)
        q = torch.empty((T, H * d), dtype=torch.float32, device=h.device)
        k = torch.empty((T, H * d), dtype=torch.float32, device=h.device)
        self.qkv_finish(proj, q, k, freq, batch, None, None, 0, 0, H, H, d, dv, k_scale, last_reader=False)
        self.retention(q, k, proj, 2 * H * d, 2 * H * d + H * dv, state, batch, decay, out, H, d, dv, eps)

    def retention(self, q, k, vg, v_off: int, g_off: int, state, batch, decay, out, H, d, dv, eps: float,
                  chunked: Optional[bool] = None) -> None:
        """The recurrence S <- decay S + k v^T, o = S^T q per head over ``state`` [slots, H, d, dv] (float32), then
        o / rms(o) * silu(g) -> out [T, H*dv].  q, k float32 [T, H*d] (rotated, k scaled); v and g are columns
        v_off.. and g_off.. of the float32 rows ``vg``.  ``chunked`` None: token by token when every request brings
        one token, chunk by chunk otherwise (and token by token where a head's state and a chunk do not fit in
        shared memory)."""
        self._need_cuda(q, k, vg, state, decay, out)
        assert q.dtype == k.dtype == vg.dtype == state.dtype == decay.dtype == torch.float32
        assert tuple(state.shape[1:]) == (H, d, dv) and decay.numel() == H and out.shape[1] == H * dv
        if chunked is None:
            chunked = batch.max_q_len > 1
        T = q.shape[0]
        ws = None
        if chunked:
            self.lib.tff_retention_workspace.restype = ctypes.c_longlong
            need = int(self.lib.tff_retention_workspace(_c_int(T), _c_int(batch.num_requests), _c_int(H), _c_int(d), _c_int(dv)))
            ws = torch.empty(need, dtype=torch.float32, device=q.device)
        clear = 1 if vg.data_ptr() in self._acc_zero else 0
        args = lambda ch: (_ptr(q), _ptr(k), _ptr(vg), _c_int(clear), _c_int(vg.shape[1]), _c_int(v_off), _c_int(g_off), _ptr(state),
                           _c_int(state.shape[0]), _ptr(batch.q_start), _ptr(batch.pos_start), _ptr(batch.slots),
                           _ptr(decay), _ptr(out), _c_int(_dt(out)), _c_int(batch.num_requests), _c_int(H), _c_int(d),
                           _c_int(dv), _c_float(eps), _c_int(ch), _ptr(ws) if ch else _vp(0), _c_int(T), self._stream())
        status = self.lib.tff_retention(*args(1 if chunked else 0))
        kernels = 3 if chunked else 1
        if status == -2 and chunked:
            status = self.lib.tff_retention(*args(0))      # a head too large for the chunked form's shared memory
            kernels = 1
        self._check(status, "retention")
        if clear:
            self._acc_zero[vg.data_ptr()] = True
        self.launches += kernels

    # ------------------------------------------------------- attention in float32 tiles (any sizes, latent caches, biases)
    @staticmethod
    def _layer_cache(kv_cache, kv_layer: int):
        """(pointer to the layer's share of the pool, elements between its pages) of a cache
        [pages, layers, planes, kv heads, page, slot], stored with the pages or with the layers outermost."""
        if not kv_cache.is_cuda:
            raise KernelError("a tensor given to a CUDA kernel is not on a CUDA device")
        st, block = kv_cache.stride(), 1
        for i in range(kv_cache.dim() - 1, 1, -1):
            if st[i] != block:
                raise KernelError("the [planes, kv heads, page, slot] block of a cache page must be dense")
            block *= kv_cache.shape[i]
        return _vp(kv_cache.data_ptr() + kv_layer * st[1] * kv_cache.element_size()), st[0]

    def attention_tile(self, q, batch, block_table, kv_cache, kv_layer, page_size, out, nq, nkv, d, dv, scale,
                       window: int = 0, chunk: int = 0, temp=None, r1=None, r2=None, out_scale: float = 1.0,
                       out_off: int = 0, num_splits=None, dense=None, softcap: float = 0.0) -> None:
        """q [T, nq*d] against the paged cache -> columns out_off .. out_off + nq*dv of ``out`` (times out_scale), in
        float32 arithmetic whatever the storage type.  The cache has two planes (keys, values) or one (the value
        of a token is the first dv elements of its key).  Visibility: causal, within ``window`` keys, within the
        query's block of ``chunk`` positions.  Scores: (q . k) * scale * temp[h] - r1[h] * ln(1 + r2[h] * distance)
        (temp, r1, r2 float32 [nq] or None); with ``softcap`` > 0 the scaled product is squashed to softcap * tanh(. / softcap)
        ahead of the distance term.  ``dense`` = (keys [T, nkv*d], values [T, nkv*dv]) of this step's own tokens
        instead of the cache: for steps whose requests all start at position 0 (bfloat16, tensor-core form only)."""
        self._need_cuda(q, block_table, out, temp, r1, r2)
        T = q.shape[0]
        assert q.dtype == out.dtype and q.shape[1] == nq * d and out.shape[0] == T and out.shape[1] >= out_off + nq * dv
        for v in (temp, r1, r2):
            assert v is None or (v.dtype == torch.float32 and v.numel() == nq)
        kd = vd = None
        if dense is not None:
            kd, vd = dense
            self._need_cuda(kd, vd)
            assert kd.dtype == vd.dtype == q.dtype and tuple(kd.shape) == (T, nkv * d) and tuple(vd.shape) == (T, nkv * dv)
            planes, slot, c_ptr, page_stride = 2, max(d, dv), _vp(0), 0
        else:
            planes, slot = kv_cache.shape[2], kv_cache.shape[-1]
            assert kv_cache.dtype == q.dtype and tuple(kv_cache.shape[3:5]) == (nkv, page_size)
            c_ptr, page_stride = self._layer_cache(kv_cache, kv_layer)
        splits = self.tile_splits(batch, nq, nkv, window, chunk) if num_splits is None else int(num_splits)
        part_o = part_ml = None
        if splits > 1:
            part_o = torch.empty(T * nq * splits * dv, dtype=torch.float32, device=q.device)
            part_ml = torch.empty(T * nq * splits * 2, dtype=torch.float32, device=q.device)
        self._check(self.lib.tff_attention_tile(
            _ptr(q), _c_int(_dt(q)), _c_int(q.shape[1]), _ptr(batch.q_start), _ptr(batch.pos_start), _ptr(block_table),
            _c_int(block_table.shape[1]), c_ptr, ctypes.c_longlong(page_stride), _c_int(planes), _c_int(page_size),
            _c_int(slot), _ptr(out), _c_int(out.shape[1]), _c_int(out_off), _c_int(batch.num_requests),
            _c_int(batch.max_q_len), _c_int(nq), _c_int(nkv), _c_int(d), _c_int(dv), _c_float(scale), _c_int(window),
            _c_int(chunk), _ptr(temp), _ptr(r1), _ptr(r2), _c_float(out_scale), _c_int(T), _c_int(splits), _ptr(part_o),
            _ptr(part_ml), _ptr(kd), _ptr(vd), _c_int(kd.shape[1] if kd is not None else 0),
            _c_int(vd.shape[1] if vd is not None else 0), _c_float(softcap), self._stream()), "attention_tile")
        self.launches += 2 if splits > 1 else 1

    def tile_splits(self, batch, nq: int, nkv: int, window: int = 0, chunk: int = 0) -> int:
        """In how many shares attention_tile cuts every tile's key range: a power of two such that a step of few rows
        behind long contexts (decoded tokens above all) still gives every SM a CTA, with at least eight key blocks
        of 32 a share (twice the shares were measured: 2.10 against 1.83 ms a step of 8 requests behind 2,048 tokens, the
        partial results' pass through memory costing more than the shorter walks save)."""
        tiles = -(-(batch.max_q_len * (nq // nkv)) // 32)
        ctas = tiles * nkv * batch.num_requests
        span = min([s for s in (window, chunk) if s > 0] + [int(batch.max_kv_len)])
        blocks = -(-span // 32)
        splits = 1
        while splits < 32 and ctas * splits * 2 <= 2 * self.NUM_SMS and splits * 2 * 4 <= blocks:
            splits *= 2
        return splits

    # ------------------------------------------------------- many small products in one launch
    def gemm_grouped(self, a, b, c, groups: int, M: int, N: int, K: int, lda: int, a_gs: int, ldb: int, b_gs: int,
                     ldc: int, c_gs: int, gated: str = "", activation: str = "silu", tiles=None, row_map=None) -> None:
        """c_g = a_g @ b_g^T ([M, K] x [N, K]^T) for ``groups`` groups whose operands lie a_gs, b_gs, c_gs elements apart
        (rows lda, ldb, ldc elements apart), float32 accumulation with a fixed order of additions.  ``gated``: b_g holds
        2N rows, gate and up, "blocked" ([N gate | N up]) or "interleaved" (alternating in blocks of 64: stack_gate_up), and
        c_g = act(a gate^T) * (a up^T).  ``tiles`` = (tile_group, tile_row0, tile_row_end, num_tiles, max_tiles, tile rows)
        is the ragged form (rows of ``a`` sorted by group, the table on the device); ``row_map`` sends product row r to
        row row_map[r] of ``c``.  bfloat16 operands of aligned sizes run on the tensor cores (csrc/gemm_grouped_mma.cu),
        everything else as float32 FMAs (csrc/gemm_grouped.cu)."""
        self._need_cuda(a, b, c, row_map)
        assert gated in ("", "blocked", "interleaved")
        tg = tr0 = tre = nt = None
        max_tiles, tile_rows = 0, 0
        if tiles is not None:
            tg, tr0, tre, nt, max_tiles, tile_rows = tiles
        code = self.ACTIVATION_CODES[activation]
        if not gated and code < 2:
            code = 0                      # a plain product: only a function of one product ("relu2") is applied to it
        act = _c_int(code)
        ll = ctypes.c_longlong
        if self.grouped_on_tensor_cores(a, b, K, lda, a_gs, ldb, b_gs, gated, N) and tile_rows in (0, self.grouped_tile_rows(True)):
            status = self.lib.tff_gemm_grouped_mma(
                _ptr(a), ll(lda), ll(a_gs), _ptr(b), ll(ldb), ll(b_gs), _ptr(c), _c_int(_dt(c)), ll(ldc), ll(c_gs),
                _ptr(tg), _ptr(tr0), _ptr(tre), _ptr(nt), _c_int(max_tiles), _ptr(row_map), _c_int(groups), _c_int(M),
                _c_int(2 * N if gated else N), _c_int(K), _c_int(1 if gated else 0), act, self._stream())
            self._check(status, "gemm_grouped_mma")
            self.launches += 1
            return
        assert tile_rows in (0, self.grouped_tile_rows(False)), "the tile table was planned for the other kernel"
        b2 = _vp(0)
        if gated:
            b2 = _vp(b.data_ptr() + (self.GATE_UP_BLOCK if gated == "interleaved" else N) * ldb * b.element_size())
        self._check(self.lib.tff_gemm_grouped(
            _ptr(a), _c_int(_dt(a)), ll(lda), ll(a_gs), _ptr(b), b2, _c_int(_dt(b)), ll(ldb), ll(b_gs),
            _ptr(c), _c_int(_dt(c)), ll(ldc), ll(c_gs), _ptr(tg), _ptr(tr0), _ptr(tre), _ptr(nt), _c_int(max_tiles),
            _ptr(row_map), _c_int(groups), _c_int(M), _c_int(N), _c_int(K), act,
            _c_int(self.GATE_UP_BLOCK if gated == "interleaved" else 0), self._stream()), "gemm_grouped")
        self.launches += 1

    GROUPED_MMA = os.environ.get("TFFINFER_GROUPED_MMA", "1") != "0"

    def grouped_on_tensor_cores(self, a, b, K, lda, a_gs, ldb, b_gs, gated: str, N: int) -> bool:
        """Whether a grouped product of these operands runs on the tensor-core kernel."""
        return (self.GROUPED_MMA and a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
                and all(v % 8 == 0 for v in (K, lda, a_gs, ldb, b_gs)) and a.data_ptr() % 16 == 0 and b.data_ptr() % 16 == 0
                and (not gated or (gated == "interleaved" and N % self.GATE_UP_BLOCK == 0)))

    def grouped_tile_rows(self, tensor_cores: bool) -> int:
        return int(self.lib.tff_gemm_grouped_mma_tile_rows() if tensor_cores else self.lib.tff_gemm_grouped_tile_rows())

    GATE_UP_BLOCK = 64       # rows of a block of the "interleaved" gate/up layout (gate_up_block above: the same)

    @classmethod
    def stack_gate_up(cls, gates, ups):
        """One tensor [E, 2*ff, W] from the experts' gate and up matrices, and the name of its layout: "interleaved"
        (64 gate rows, the 64 up rows of the same outputs, ...: what the tensor-core kernels' epilogues want, as
        merge_gate_up lays out a dense feed-forward) when ff is a multiple of 64, else "blocked" (all gate rows, then
        all up rows)."""
        g, u = torch.stack(list(gates), dim=0), torch.stack(list(ups), dim=0)
        E, ff, W = g.shape
        b = cls.GATE_UP_BLOCK
        if ff % b == 0:
            w = torch.stack([g.view(E, ff // b, b, W), u.view(E, ff // b, b, W)], dim=2).reshape(E, 2 * ff, W)
            return w.contiguous(), "interleaved"
        return torch.cat([g, u], dim=1).contiguous(), "blocked"

    # ------------------------------------------------------- short convolutions, hashed pair embedding, plain activations
    def short_conv_norm(self, proj, out, segments, taps: int, eps: float, state, batch) -> None:
        """A causal convolution of ``taps`` taps over time on column segments of the float32 rows ``proj`` [T, ld] and the
        RMS norm of whole segments behind it -> ``out`` [T, ld] float32 (columns beyond the segments are copied).
        ``segments``: up to three (width, conv weights float32 [width, taps] or None, norm weight float32 [width] or
        None), lying one behind the other from column 0.  ``state`` [slots, taps-1, C] float32 holds every request's
        last taps-1 rows of the segments from earlier steps (csrc/short_conv.cu); short_conv_state updates it."""
        self._need_cuda(proj, out, state)
        T, ld = proj.shape
        n = len(segments)
        assert proj.dtype == out.dtype == torch.float32 and tuple(out.shape) == (T, ld) and 1 <= n <= 3
        C = sum(int(w) for w, _, _ in segments)
        for width, cw, nw in segments:
            self._need_cuda(cw, nw)
            assert cw is None or (cw.dtype == torch.float32 and tuple(cw.shape) == (width, taps))
            assert nw is None or (nw.dtype == torch.float32 and nw.numel() == width)
        if taps > 1:
            assert state is not None and state.dtype == torch.float32 and tuple(state.shape[1:]) == (taps - 1, C)
        widths = (_c_int * n)(*[int(w) for w, _, _ in segments])
        convs = (_vp * n)(*[cw.data_ptr() if cw is not None else None for _, cw, _ in segments])
        norms = (_vp * n)(*[nw.data_ptr() if nw is not None else None for _, _, nw in segments])
        self._check(self.lib.tff_short_conv_norm(_ptr(proj), _c_int(ld), _ptr(out), _c_int(n), widths, convs, norms,
                                                 _c_int(taps), _c_float(eps), _ptr(state), _ptr(batch.positions),
                                                 _ptr(batch.tok_req), _ptr(batch.q_start), _ptr(batch.slots), _c_int(T),
                                                 self._stream()), "short_conv_norm")
        self.launches += 1

    CONV_FINISH = os.environ.get("TFFINFER_CONV_FINISH", "1") != "0"   # 0: the convolution and the finish as two kernels

    def conv_finish(self, proj, conv, norm, taps: int, eps: float, state, q_out, freq, batch, block_table, kv_cache,
                    kv_layer, page_size, nq, nkv, d, dv, gate_off: int = -1, gate_out=None) -> None:
        """short_conv_norm and qkv_finish in one kernel (csrc/short_conv.cu conv_finish_kernel): the float32 rows ``proj``
        [T, ld] = [q | k | v | gates ...] are convolved over time (``conv`` = three float32 [taps, width], the weights
        transposed so that a tap's weights of neighbouring channels lie together, or None), q and k
        normed over their whole width (``norm`` = two float32 [width] or None), rotated (``freq`` as for qkv_finish) and
        stored: q to ``q_out`` [T, nq*d], k and v to the tokens' cache slots, the sigmoid of the gates to ``gate_out``.
        ``proj`` is left as it is: short_conv_state, behind it, keeps the rows the next step needs and clears them."""
        self._need_cuda(proj, q_out, state, block_table, gate_out)
        T, ld = proj.shape
        assert proj.dtype == torch.float32 and kv_cache is not None and tuple(kv_cache.shape[2:5]) == (2, nkv, page_size)
        widths = (nq * d, nkv * d, nkv * dv)
        for width, cw in zip(widths, conv):
            self._need_cuda(cw)
            assert cw is None or (cw.dtype == torch.float32 and tuple(cw.shape) == (taps, width) and cw.is_contiguous())
        for width, nw in zip(widths, norm):
            self._need_cuda(nw)
            assert nw is None or (nw.dtype == torch.float32 and nw.numel() == width)
        if taps > 1:
            assert state is not None and state.dtype == torch.float32 and tuple(state.shape[1:]) == (taps - 1, sum(widths))
        f, rot, mag, inter = freq if freq is not None else (None, 0, 1.0, False)
        c_ptr, _, c_layers, c_layer = self._cache_args(kv_cache, kv_layer)
        convs = (_vp * 3)(*[cw.data_ptr() if cw is not None else None for cw in conv])
        norms = (_vp * 2)(*[nw.data_ptr() if nw is not None else None for nw in norm])
        self._check(self.lib.tff_conv_finish(
            _ptr(proj), _c_int(ld), convs, norms, _c_int(taps), _c_float(eps), _ptr(state), _ptr(batch.positions),
            _ptr(batch.tok_req), _ptr(batch.q_start), _ptr(batch.slots), _ptr(q_out), _c_int(_dt(q_out)), _ptr(f), _c_int(rot),
            _c_float(mag), _c_int(1 if inter else 0), _ptr(block_table), _c_int(block_table.shape[1]), c_ptr,
            _c_int(_dt(kv_cache)), _c_int(c_layers), _c_int(c_layer), _c_int(page_size), _c_int(kv_cache.shape[-1]),
            _c_int(gate_off), _ptr(gate_out), _c_int(T), _c_int(nq), _c_int(nkv), _c_int(d), _c_int(dv), self._stream()),
            "conv_finish")
        self.launches += 1

    def short_conv_state(self, proj, taps: int, channels: int, state, batch) -> None:
        """Behind short_conv_norm: every request's last taps-1 rows of the first ``channels`` columns of ``proj`` go to its
        slot of ``state`` (older rows move up when the portion is shorter).  When ``proj`` is one of the accumulator
        buffers that are kept at zero between uses, its rows are set back to zero."""
        self._need_cuda(proj, state)
        clear = 1 if proj.data_ptr() in self._acc_zero else 0
        if taps <= 1 and not clear:
            return
        self._check(self.lib.tff_short_conv_state(_ptr(proj), _c_int(proj.shape[1]), _c_int(clear), _c_int(taps),
                                                  _c_int(channels), _ptr(state), _ptr(batch.q_start), _ptr(batch.pos_start),
                                                  _ptr(batch.slots), _c_int(batch.num_requests), self._stream()),
                    "short_conv_state")
        if clear:
            self._acc_zero[proj.data_ptr()] = True
        self.launches += 1

    def pair_embed(self, batch, state, table, buckets: int, mul_prev: int, mul_cur: int, x, copies: int = 0) -> None:
        """x[t] += table[(prev * mul_prev + token * mul_cur) mod buckets], prev the token before t in its request; row
        ``buckets`` for a request's first token.  ``state`` int32 [slots, 1] holds every request's last token of earlier
        steps and is updated.  x float32 [T, W], or [T, copies, W] with every copy getting the row."""
        self._need_cuda(state, table, x)
        W = x.shape[-1]
        assert state.dtype == torch.int32 and x.dtype == torch.float32 and tuple(table.shape) == (buckets + 1, W)
        assert x.shape[0] == batch.num_tokens and (copies == 0 or x.shape[1] == copies)
        ll = ctypes.c_longlong
        self._check(self.lib.tff_pair_embed(_ptr(batch.token_ids), _ptr(batch.positions), _ptr(batch.tok_req),
                                            _ptr(batch.q_start), _ptr(batch.slots), _ptr(state), _ptr(table),
                                            _c_int(_dt(table)), _c_int(buckets), ll(mul_prev), ll(mul_cur), _ptr(x),
                                            _c_int(max(copies, 1)), _c_int(W), _c_int(batch.num_tokens),
                                            _c_int(batch.num_requests), self._stream()), "pair_embed")
        self.launches += 2

    def unary_act(self, x, out, activation: str) -> None:
        """out = act(x) element by element (may be in place; x float32 and out bfloat16 also); act "relu2": the square
        of relu.  An x that is one of the accumulator buffers kept at zero between uses is cleared behind the read."""
        self._need_cuda(x, out)
        assert x.numel() == out.numel() and (x.dtype == out.dtype or x.dtype == torch.float32)
        clear = 1 if (x.data_ptr() in self._acc_zero and x.data_ptr() != out.data_ptr()) else 0
        self._check(self.lib.tff_unary_act(_ptr(x), _c_int(_dt(x)), _ptr(out), _c_int(_dt(out)), ctypes.c_longlong(x.numel()),
                                           _c_int(self.ACTIVATION_CODES[activation]), _c_int(clear), self._stream()), "unary_act")
        if clear:
            self._acc_zero[x.data_ptr()] = True
        self.launches += 1

    def gemm_act(self, a, w, out, activation: str = "relu2") -> None:
        """out[T, N] = act(a @ w^T) for an activation of one product ("relu2").  Above CLUSTER_MAX_M rows in bfloat16 the
        activation is applied in the tcgen05 product's epilogue; decode-sized and float32 steps run the product into
        float32 and the activation kernel behind it."""
        self._need_cuda(a, w, out)
        T, N = out.shape
        K = a.shape[1]
        tc = (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and K % 8 == 0 and a.data_ptr() % 16 == 0
              and w.data_ptr() % 16 == 0)
        if tc and T > self.CLUSTER_MAX_M and N % 8 == 0 and out.dtype == torch.bfloat16 and out.data_ptr() % 16 == 0:
            bn = self.prompt_plan(T, N, K, False, kinds=(256, 128))[1]
            self._check(self.lib.tff_gemm_tc_act(_ptr(a), _ptr(w), _ptr(out), _c_int(T), _c_int(N), _c_int(K), _c_int(bn),
                                                 _c_int(self.ACTIVATION_CODES[activation]), self._stream()), "gemm_tc_act")
            self.launches += 1
            return
        if tc and T <= self.SWAP_MAX_M:
            up = self.projection_buffer(T, N, out.device, out.dtype, use="act")
        else:
            up = torch.empty((T, N), dtype=torch.float32, device=out.device)
        self.gemm(a, w, up)
        self.unary_act(up, out, activation)

    def plain_mlp(self, h, w_up, w_down, residual, activation: str = "relu2", out=None) -> None:
        """residual += down(act(up(h))), a feed-forward without a gate; with ``residual`` None the result goes to ``out``."""
        if isinstance(h, DeferredNorm):
            h = h.materialize()
        act = torch.empty((h.shape[0], w_up.shape[0]), dtype=h.dtype, device=h.device)
        self.gemm_act(h, w_up, act, activation)
        if residual is None:
            self.gemm(act, w_down, out)
        else:
            self.gemm(act, w_down, residual, residual=residual)

    # ------------------------------------------------------- routed feed-forward (mixture of experts)
    def routed_mlp(self, h, w_router, w_gate_up, layout: str, w_down, residual, top: int, renormalize: bool = False,
                   weight_on: str = "output", activation: str = "silu", out=None, router=None) -> None:
        """residual += sum over a token's ``top`` experts of down_e(act(gate_e(x)) * up_e(x)), the experts chosen by
        the largest sigmoid(W_r h) (computed in float32), weights the scores themselves or renormalised to sum 1;
        ``weight_on`` "input": x = w h and the outputs are summed as they are; "output": x = h and the outputs are
        summed with the weights.  (w_gate_up, layout) = stack_gate_up(...) [E, 2*ff, W], w_down [E, W, ff].  With
        ``layout`` "plain" the experts are not gated: w_gate_up is [E, ff, W] and an expert is down_e(act(up_e(x))) with
        ``activation`` a function of one product ("relu2").  ``router`` (see moe_dispatch): softmax scores, a correction of
        the choice, groups of experts, identity experts (router outputs beyond the E experts: weight times the input).
        With ``residual`` None the sum goes to ``out``.  Six launches, no host synchronisation: route, plan, gather, two
        grouped products over the tokens sorted by expert, combine (a token's experts are added in the order of their
        rank)."""
        if isinstance(h, DeferredNorm):
            h = h.materialize()
        self._need_cuda(h, w_router, w_gate_up, w_down, residual, out)
        T, W = h.shape
        plain = layout == "plain"
        E, ff = w_gate_up.shape[0], (w_gate_up.shape[1] if plain else w_gate_up.shape[1] // 2)
        up_rows = ff if plain else 2 * ff
        identity = int((router or {}).get("identity", 0))
        assert tuple(w_router.shape) == (E + identity, W) and tuple(w_gate_up.shape) == (E, up_rows, W)
        assert tuple(w_down.shape) == (E, W, ff)
        assert weight_on in ("input", "output") and 0 < top <= E + identity
        if plain and activation not in ("relu2",):
            raise KernelError(f"experts that are not gated take the activation 'relu2', got '{activation}'")
        if not plain and activation not in ("silu", "gelu_tanh"):
            raise KernelError(f"gated experts take the activations 'silu' and 'gelu_tanh', got '{activation}'")
        target = residual if residual is not None else out
        assert target.dtype == torch.float32 and tuple(target.shape) == (T, W)
        P = T * top
        # both products run on the same kernel (one tile table): the tensor-core one if both can
        tc = (self.grouped_on_tensor_cores(h, w_gate_up, W, W, 0, W, up_rows * W, "" if plain else layout, ff)
              and self.grouped_on_tensor_cores(h, w_down, ff, ff, 0, ff, W * ff, "", W))
        if tc and self.GROUPED_TCGEN05 and P >= self.GROUPED_TCGEN05_FROM and W % 4 == 0 and ff % 8 == 0:
            # Prompt-sized: the tcgen05 product in its grouped form.  Every expert's rows are padded to whole tiles of 128
            # in the sorted order, both products write in that order, and the sum gathers a token's rows from it.
            rows = -(-(P + E * 127) // 128) * 128
            pair_weight, row_map, tiles, x, lane_group, place, *pe = self.moe_dispatch(
                h, w_router, top, renormalize, weight_on == "input", 128, padded_rows=rows, router=router)
            act = torch.empty((rows, ff), dtype=h.dtype, device=h.device)
            self.gemm_tc_grouped(x, w_gate_up, act, E, up_rows, W, lane_group, gated=not plain, activation=activation)
            y = torch.empty((rows, W), dtype=torch.float32, device=h.device)
            self.gemm_tc_grouped(act, w_down, y, E, W, ff, lane_group)
            self.moe_combine(y, pair_weight if weight_on == "output" else None, top, residual, target, place,
                             identity=(pe[0], pair_weight, h) if pe else None)
            return
        pair_weight, row_map, tiles, x, *pe = self.moe_dispatch(h, w_router, top, renormalize, weight_on == "input",
                                                                self.grouped_tile_rows(tc), router=router)
        act = torch.empty((P, ff), dtype=h.dtype, device=h.device)
        self.gemm_grouped(x, w_gate_up, act, E, 0, ff, W, W, 0, W, up_rows * W, ff, 0, gated="" if plain else layout,
                          activation=activation, tiles=tiles)
        y = torch.empty((P, W), dtype=torch.float32, device=h.device)
        self.gemm_grouped(act, w_down, y, E, 0, W, ff, ff, 0, ff, W * ff, W, 0, tiles=tiles, row_map=row_map)
        self.moe_combine(y, pair_weight if weight_on == "output" else None, top, residual, target,
                         identity=(pe[0], pair_weight, h) if pe else None)

    GROUPED_TCGEN05 = os.environ.get("TFFINFER_GROUPED_TCGEN05", "1") != "0"
    GROUPED_TCGEN05_FROM = 1024      # (token, expert) pairs of a step from which the experts run on the tcgen05 product

    def gemm_tc_grouped(self, a, w, out, groups: int, group_rows: int, K: int, lane_group, gated: bool = False,
                        activation: str = "silu") -> None:
        """out = a @ w_g^T tile by tile of 128 rows of ``a``, tile t with group lane_group[t] (int32 on the device, -1: no
        such tile) of ``w`` [groups, group_rows, K]; gated: w_g holds gate and up rows alternating in blocks of 64 and
        out has group_rows / 2 columns.  The tcgen05 product of csrc/gemm_tc.cu in its grouped form."""
        self._need_cuda(a, w, out, lane_group)
        rows = a.shape[0]
        assert a.dtype == w.dtype == torch.bfloat16 and a.shape[1] == K and rows % 128 == 0 and lane_group.numel() >= rows // 128
        assert tuple(w.shape) == (groups, group_rows, K) and out.shape[0] == rows
        assert out.shape[1] == (group_rows // 2 if gated else group_rows)
        bn = 256 if (group_rows % 256 == 0 and rows >= 2048) else 128
        code = self.ACTIVATION_CODES[activation]
        if not gated and code < 2:
            code = 0                      # a plain product: only a function of one product ("relu2") is applied to it
        self._check(self.lib.tff_gemm_tc_grouped(_ptr(a), _ptr(w), _ptr(out), _c_int(_dt(out)), _c_int(rows), _c_int(groups),
                                                 _c_int(group_rows), _c_int(K), _c_int(bn), _c_int(1 if gated else 0),
                                                 _c_int(code), _ptr(lane_group), self._stream()), "gemm_tc_grouped")
        self.launches += 1

    def moe_dispatch(self, h, w_router, top: int, renormalize: bool, scale_rows: bool, tile_rows: int = 0,
                     padded_rows: int = 0, router=None):
        """Router, choice and sorting of a routed feed-forward (csrc/moe.cu: route, plan, gather).  Returns
        (pair_weight float32 [T*top], row_map int32 [T*top]: sorted place -> pair, the tile table of the grouped
        products, x [T*top, W]: the tokens' rows sorted by expert, times their weight when ``scale_rows``).  With
        ``padded_rows`` (a multiple of ``tile_rows``, at least T*top + E*(tile_rows-1)) every expert's rows start at a
        multiple of ``tile_rows``, x has that many rows, and two more are returned: lane_group (int32, the expert of
        every tile of x, -1 for tiles nobody uses) and place_of_pair (int32 [T*top]).  ``router`` = dict(score="sigmoid" |
        "softmax" | "softmax_chosen" (the logits choose, the chosen are weighted by a softmax among themselves),
        bias=float32 [outputs] or None (added to the logits), correction=float32 [outputs] or None, groups=(count, keep), identity=n): the router's last n outputs are
        identity experts, whose pairs get no row (pair_expert -1; returned as a last, further value when n > 0)."""
        T, W = h.shape
        r = router or {}
        identity = int(r.get("identity", 0))
        E = w_router.shape[0] - identity                          # experts that have rows
        groups, keep = r.get("groups") or (1, 1)
        correction = r.get("correction")
        self._need_cuda(correction)
        assert correction is None or (correction.dtype == torch.float32 and correction.numel() == E + identity)
        dev, P = h.device, T * top
        counts = self._moe_counts.get((E, str(dev)))
        if counts is None:
            counts = torch.zeros(E, dtype=torch.int32, device=dev)       # set back to zero by the plan kernel
            self._moe_counts[(E, str(dev))] = counts
        bm = tile_rows or self.grouped_tile_rows(False)      # rows of a tile of the grouped product that follows
        max_tiles = -(-P // bm) + E
        R = max(P, padded_rows)                              # rows of the sorted order
        lane_tiles = padded_rows // bm if padded_rows else 0
        ints = torch.empty(P + R + E + 3 * max_tiles + 1 + lane_tiles + (P if padded_rows else 0), dtype=torch.int32, device=dev)
        pair_expert, row_map, cursor = ints[:P], ints[P:P + R], ints[P + R:P + R + E]
        o = P + R + E
        tile_group, tile_row0, tile_row_end = ints[o:o + max_tiles], ints[o + max_tiles:o + 2 * max_tiles], ints[o + 2 * max_tiles:o + 3 * max_tiles]
        num_tiles = ints[o + 3 * max_tiles:o + 3 * max_tiles + 1]
        lane_group = ints[o + 3 * max_tiles + 1:o + 3 * max_tiles + 1 + lane_tiles] if padded_rows else None
        place = ints[o + 3 * max_tiles + 1 + lane_tiles:] if padded_rows else None
        pair_weight = torch.empty(P, dtype=torch.float32, device=dev)
        bias = r.get("bias")
        self._need_cuda(bias)
        assert bias is None or (bias.dtype == torch.float32 and bias.numel() == E + identity)
        self._check(self.lib.tff_moe_route(_ptr(h), _c_int(_dt(h)), _ptr(w_router), _c_int(_dt(w_router)), _ptr(bias), _c_int(T), _c_int(W),
                                           _c_int(E + identity), _c_int(top), _c_int(1 if renormalize else 0),
                                           _c_int({"sigmoid": 0, "softmax": 1, "softmax_chosen": 2}[r.get("score", "sigmoid")]), _ptr(correction),
                                           _c_int(int(groups)), _c_int(int(keep)), _c_int(E), _ptr(pair_expert),
                                           _ptr(pair_weight), _ptr(counts), self._stream()), "moe_route")
        self._check(self.lib.tff_moe_plan(_ptr(counts), _c_int(E), _c_int(bm), _ptr(cursor), _ptr(tile_group), _ptr(tile_row0),
                                          _ptr(tile_row_end), _ptr(num_tiles), _c_int(bm if padded_rows else 0),
                                          _ptr(lane_group), _c_int(lane_tiles), self._stream()), "moe_plan")
        x = torch.empty((R, W), dtype=h.dtype, device=dev)
        self._check(self.lib.tff_moe_gather(_ptr(h), _c_int(_dt(h)), _c_int(P), _c_int(W), _c_int(top), _ptr(pair_expert),
                                            _ptr(pair_weight), _c_int(1 if scale_rows else 0), _ptr(cursor),
                                            _ptr(row_map), _ptr(place), _ptr(x), self._stream()), "moe_gather")
        self.launches += 3
        tiles = (tile_group, tile_row0, tile_row_end, num_tiles, max_tiles, bm)
        extra = (pair_expert,) if identity else ()
        if padded_rows:
            return (pair_weight, row_map, tiles, x, lane_group, place) + extra
        return (pair_weight, row_map, tiles, x) + extra

    def moe_combine(self, y, pair_weight, top: int, residual, out, place_of_pair=None, identity=None) -> None:
        """out[t] = residual[t] + sum_k w[t, k] * y[t*top + k] in the order of k (pair_weight None: plain sum); with
        ``place_of_pair`` the row of pair t*top + k is y[place_of_pair[t*top + k]] (y in the sorted order).  ``identity`` =
        (pair_expert, pair_weight, h): pairs whose expert is -1 add their weight times the token's row of ``h`` instead."""
        T, W = out.shape
        pe, iw, h = identity if identity is not None else (None, None, None)
        if identity is not None and pair_weight is None:
            weights, on_output = iw, 0            # the weights are read for the identity pairs only
        else:
            weights, on_output = pair_weight, 1 if pair_weight is not None else 0
        self._check(self.lib.tff_moe_combine(_ptr(y), _c_int(T), _c_int(W), _c_int(top), _ptr(weights),
                                             _c_int(on_output), _ptr(place_of_pair),
                                             _ptr(residual), _ptr(out), _ptr(pe), _ptr(h),
                                             _c_int(_dt(h)) if h is not None else _c_int(0), self._stream()), "moe_combine")
        self.launches += 1

    # ------------------------------------------------------- gated recurrence over a state of one vector
    def min_gru(self, proj, z_off: int, x_off: int, g_off: int, bz, bx, state, batch, out, width: int, out_off: int = 0,
                out_scale: float = 1.0, last_reader: bool = True) -> None:
        """The minGRU recurrence (csrc/mingru.cu) from columns z_off.., x_off.., g_off.. of the float32 rows ``proj``
        over ``state`` [slots, width] -> columns out_off .. out_off + width of ``out`` (times out_scale)."""
        self._need_cuda(proj, bz, bx, state, out)
        assert proj.dtype == torch.float32 and state.dtype == torch.float32 and state.shape[1] == width
        assert out.shape[0] == proj.shape[0] and out.shape[1] >= out_off + width
        for v in (bz, bx):
            assert v is None or (v.dtype == torch.float32 and v.numel() == width)
        clear = 1 if proj.data_ptr() in self._acc_zero else 0
        if batch.max_q_len > self.GRU_CHUNKED_FROM:
            # long portions: chunks of a request side by side (three passes), not one thread walking thousands of tokens
            self.lib.tff_min_gru_workspace.restype = ctypes.c_longlong
            need = int(self.lib.tff_min_gru_workspace(_c_int(batch.num_requests), _c_int(batch.max_q_len), _c_int(width)))
            ws = torch.empty(need, dtype=torch.float32, device=proj.device)
            self._check(self.lib.tff_min_gru_chunked(
                _ptr(proj), _c_int(proj.shape[1]), _c_int(z_off), _c_int(x_off), _c_int(g_off), _c_int(clear), _ptr(bz),
                _ptr(bx), _ptr(state), _c_int(state.shape[0]), _ptr(batch.q_start), _ptr(batch.slots),
                _c_int(batch.num_requests), _c_int(batch.max_q_len), _c_int(width), _ptr(ws), _ptr(out), _c_int(_dt(out)),
                _c_int(out.shape[1]), _c_int(out_off), _c_float(out_scale), self._stream()), "min_gru_chunked")
            self.launches += 3
        else:
            self._check(self.lib.tff_min_gru(_ptr(proj), _c_int(proj.shape[1]), _c_int(z_off), _c_int(x_off), _c_int(g_off),
                                             _c_int(clear), _ptr(bz), _ptr(bx), _ptr(state), _c_int(state.shape[0]),
                                             _ptr(batch.q_start), _ptr(batch.slots), _c_int(batch.num_requests), _c_int(width),
                                             _ptr(out), _c_int(_dt(out)), _c_int(out.shape[1]), _c_int(out_off),
                                             _c_float(out_scale), self._stream()), "min_gru")
            self.launches += 1
        if clear and last_reader:
            self._acc_zero[proj.data_ptr()] = True

    GRU_CHUNKED_FROM = 32         # longest portion of a step from which the recurrence runs chunk by chunk

    # ------------------------------------------------------- recurrences over a matrix state with a decay read from the input
    def linear_recurrence(self, q, k, v, dec, state, batch, out, H: int, K: int, V: int, mode: str, share: int = 1,
                          dec_bias=None, rate_log=None, skip=None, inv_tau: float = 1.0, q_scale: float = 1.0,
                          state_off: int = 0) -> None:
        """S_t = diag(a_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t (+ skip_h v_t) per head over a float32 state [K, V]
        (csrc/linear_recurrence.cu).  q, k, v, dec are (float32 rows [T, ld], first column): column blocks of a
        projection's accumulators or tensors of their own; ``share`` heads use one q and one k.  ``mode``: "log" (dec =
        ln a per key channel), "gate" (a = sigmoid(dec + dec_bias)^inv_tau per key channel), "step" (dt = softplus(dec +
        dec_bias) per head, a = exp(-exp(rate_log) dt), k times dt).  ``state`` [slots, n] float32: a request's heads lie
        at elements state_off .. of its slot.  out float32 [T, H*V].  Two kernels: the decay factors of all tokens, once,
        then the walk over the tokens; portions of more than 256 tokens are walked as segments side by side, which a scan
        over the segments' states and a kernel that adds what every token still lacks join (two kernels more)."""
        (qt, q0), (kt, k0), (vt, vo), (dt, d0) = q, k, v, dec
        self._need_cuda(qt, kt, vt, dt, state, out, dec_bias, rate_log, skip)
        for t in (qt, kt, vt, dt, state, out):
            assert t.dtype == torch.float32
        assert state.dim() == 2 and state_off + H * K * V <= state.shape[1] and tuple(out.shape) == (qt.shape[0], H * V)
        G = H // share
        assert H % share == 0 and q0 + G * K <= qt.shape[1] and k0 + G * K <= kt.shape[1] and vo + H * V <= vt.shape[1]
        m = {"log": 0, "gate": 1, "step": 2}[mode]
        assert d0 + (H if m == 2 else H * K) <= dt.shape[1]
        for t, n in ((dec_bias, H if m == 2 else H * K), (rate_log, H), (skip, H)):
            assert t is None or (t.dtype == torch.float32 and t.numel() == n)
        T = qt.shape[0]
        self.lib.tff_linear_recurrence_workspace.restype = ctypes.c_longlong
        need = int(self.lib.tff_linear_recurrence_workspace(_c_int(T), _c_int(batch.num_requests), _c_int(batch.max_q_len),
                                                            _c_int(H), _c_int(K), _c_int(V), _c_int(m)))
        factors = torch.empty(need, dtype=torch.float32, device=qt.device)
        segmented = batch.max_q_len > self.RECURRENCE_SEGMENT
        self._check(self.lib.tff_linear_recurrence(
            _ptr(qt), _c_int(qt.shape[1]), _c_int(q0), _ptr(kt), _c_int(kt.shape[1]), _c_int(k0), _ptr(vt),
            _c_int(vt.shape[1]), _c_int(vo), _ptr(dt), _c_int(dt.shape[1]), _c_int(d0), _ptr(dec_bias), _ptr(rate_log),
            _ptr(skip), _c_int(m), _c_float(inv_tau), _c_float(q_scale), _ptr(state), ctypes.c_longlong(state.shape[1]),
            ctypes.c_longlong(state_off), _ptr(batch.q_start), _ptr(batch.pos_start), _ptr(batch.slots), _ptr(out),
            _c_int(out.shape[1]), _ptr(factors), _c_int(T), _c_int(batch.num_requests), _c_int(batch.max_q_len), _c_int(H),
            _c_int(K), _c_int(V), _c_int(share), self._stream()), "linear_recurrence")
        self.launches += 4 if segmented else 2

    RECURRENCE_SEGMENT = 256      # portions longer than this run as segments side by side, joined by a scan (the kernel's constant)

    def gated_norm(self, o, group: int, gate, gate_off: int, weight, eps: float, gate_first: bool, out, out_off: int = 0,
                   out_scale: float = 1.0, clear_cols=None, last_reader: bool = False) -> None:
        """o float32 [T, width] in groups of ``group`` columns: RMS norm of every group times weight[c mod len(weight)]
        and the silu of columns gate_off .. of the float32 rows ``gate``, the gate ahead of the norm (``gate_first``) or
        behind it -> columns out_off .. of ``out`` times out_scale.  ``clear_cols`` = (lo, hi): when ``gate`` is one of
        the accumulator buffers kept at zero between uses, those columns of it are set back to zero; ``last_reader``
        says that nothing else of its rows is left unread, so that the buffer counts as clean again."""
        self._need_cuda(o, gate, weight, out)
        T, width = o.shape
        assert o.dtype == gate.dtype == weight.dtype == torch.float32 and width % group == 0
        assert gate_off + width <= gate.shape[1] and out.shape[0] == T and out_off + width <= out.shape[1]
        clear = 1 if (clear_cols is not None and gate.data_ptr() in self._acc_zero) else 0
        lo, hi = clear_cols if clear_cols is not None else (0, 0)
        self._check(self.lib.tff_gated_norm(
            _ptr(o), _c_int(width), _c_int(group), _ptr(gate), _c_int(gate.shape[1]), _c_int(gate_off), _ptr(weight),
            _c_int(weight.numel()), _c_float(eps), _c_int(1 if gate_first else 0), _ptr(out), _c_int(_dt(out)),
            _c_int(out.shape[1]), _c_int(out_off), _c_float(out_scale), _c_int(clear), _c_int(lo), _c_int(hi), _c_int(T),
            self._stream()), "gated_norm")
        if clear and last_reader:
            self._acc_zero[gate.data_ptr()] = True
        self.launches += 2 if clear and hi > lo else 1

    def causal_conv(self, proj, col0: int, channels: int, weight, bias, activation: str, state, state_off: int, batch,
                    out, update_state: bool = False) -> bool:
        """y[t, c] = act(bias[c] + sum_j weight[c, j] u[t - taps + 1 + j, c]) over columns col0 .. col0 + channels of the
        float32 rows ``proj`` -> out float32 [T, channels]; the rows ahead of a request's portion come from elements
        state_off .. of its slot of ``state`` [slots, n] ([taps-1, channels], oldest first), zeros ahead of position 0.
        ``causal_conv_state`` behind it keeps the rows the next step needs; in a step in which every request brings one
        token ``update_state`` lets this kernel do that itself; returns whether it did."""
        self._need_cuda(proj, weight, bias, state, out)
        T = proj.shape[0]
        taps = weight.shape[1]
        assert proj.dtype == weight.dtype == out.dtype == torch.float32 and tuple(weight.shape) == (channels, taps)
        assert tuple(out.shape) == (T, channels) and (bias is None or (bias.dtype == torch.float32 and bias.numel() == channels))
        assert taps == 1 or (state is not None and state.dtype == torch.float32 and state.dim() == 2
                             and state_off + (taps - 1) * channels <= state.shape[1])
        fused = bool(update_state) and batch.max_q_len == 1 and taps > 1
        self._check(self.lib.tff_causal_conv(
            _ptr(proj), _c_int(proj.shape[1]), _c_int(col0), _c_int(channels), _ptr(weight), _ptr(bias), _c_int(taps),
            _c_int({"none": 0, "silu": 1}[activation]), _ptr(state), ctypes.c_longlong(state.shape[1] if state is not None else 0),
            ctypes.c_longlong(state_off), _ptr(batch.positions), _ptr(batch.tok_req), _ptr(batch.q_start), _ptr(batch.slots),
            _ptr(out), _c_int(T), _c_int(1 if fused else 0), self._stream()), "causal_conv")
        self.launches += 1
        return fused

    def causal_conv_state(self, proj, col0: int, channels: int, taps: int, state, state_off: int, batch) -> None:
        """Every request's last taps-1 rows of columns col0 .. col0 + channels of ``proj`` go to its slot (older rows move
        up when the portion is shorter)."""
        if taps <= 1:
            return
        self._need_cuda(proj, state)
        self._check(self.lib.tff_causal_conv_state(
            _ptr(proj), _c_int(proj.shape[1]), _c_int(col0), _c_int(channels), _c_int(taps), _ptr(state),
            ctypes.c_longlong(state.shape[1]), ctypes.c_longlong(state_off), _ptr(batch.q_start), _ptr(batch.slots),
            _c_int(batch.num_requests), self._stream()), "causal_conv_state")
        self.launches += 1

    # ------------------------------------------------------- latent attention
    PER_HEAD_FROM = 128       # longest portion of a step of whole prompts from which a latent attention makes per-head keys

    def latent_attend(self, h, w_down, q_norm_w, kv_norm_w, eps: float, w_uq, w_uk_t, w_uv, freq, batch, block_table,
                      kv_cache, kv_layer, page_size, out, heads: int, dim: int, rot_dim: int, vdim: int, q_rank: int,
                      kv_rank: int, scale: float, write_cache: bool, w_uk=None, shared=None) -> None:
        """The whole of a latent attention between its input rows and its output projection -> out [T, heads*vdim].
        ``w_down`` rows [query latent (q_rank) | kv latent (kv_rank) | shared rotated key part (rot_dim)], the last two
        absent when the layer reads another layer's cache (``write_cache`` False).  The cache has one plane with a slot
        [c | r] of kv_rank + rot_dim elements per token.  Per-head keys W_uk c are never made: the query's unrotated
        part goes through W_uk^T instead (``w_uk_t`` [heads, kv_rank, dim]), attention then runs with one shared
        key/value head over the slots (keys the whole slot, values its first kv_rank elements), and W_uv [heads*vdim,
        kv_rank] takes every head's mixed latent to its value size.

        A step of whole prompts (every request starts at position 0, bfloat16, aligned sizes) takes the other form: the
        step's latents are also kept in plain rows (``shared``, a dict that lives for the step, hands them to the layers
        that read this layer's cache), per-head keys [W_uk c | r] and values W_uv c of the step's tokens are made by
        grouped products (``w_uk`` [heads*dim, kv_rank]), and attention runs with keys of dim + rot_dim and values of
        vdim elements: a fifth of the absorbed form's arithmetic at the sizes of a large model.  The cache is written
        either way."""
        if isinstance(h, DeferredNorm):
            h = h.materialize()
        T = h.shape[0]
        dev, dt = h.device, h.dtype
        slot = kv_rank + rot_dim
        whole = (dt == torch.bfloat16 and shared is not None and getattr(batch, "h_pos_start", None) is not None
                 and batch.max_q_len >= self.PER_HEAD_FROM and not np.any(batch.h_pos_start[:batch.num_requests])
                 and slot % 8 == 0 and kv_rank % 8 == 0)
        key = ("latent rows", kv_cache.data_ptr(), kv_layer)
        assert kv_cache is not None and kv_cache.shape[2] == 1 and kv_cache.shape[3] == 1 and kv_cache.shape[-1] == slot
        assert w_down.shape[0] >= (q_rank + slot if write_cache else q_rank)      # rows beyond are padding
        f, rot_dims, mag, inter = freq if freq is not None else (None, 0, 1.0, True)
        if rot_dims and (not inter or mag != 1.0):
            raise KernelError("latent attention turns interleaved pairs by plain angles")
        proj = self.projection_buffer(T, w_down.shape[0], dev, dt)
        self.gemm(h, w_down, proj)
        cq = torch.empty((T, q_rank), dtype=dt, device=dev)
        rows = None
        if whole and write_cache:
            rows = shared[key] = torch.empty((T, slot), dtype=dt, device=dev)
        elif whole:
            rows = shared.get(key)
        self.latent_finish(proj, cq, q_norm_w, kv_norm_w, eps, f, rot_dim, rot_dims, batch, block_table, kv_cache, kv_layer,
                           page_size, q_rank, kv_rank if write_cache else 0, dense_out=rows if write_cache else None)
        q = torch.empty((T, heads * (dim + rot_dim)), dtype=dt, device=dev)
        self.gemm(cq, w_uq, q)
        if (rows is not None and w_uk is not None and (dim + rot_dim) % 8 == 0 and vdim % 8 == 0
                and tuple(rows.shape) == (T, slot)):
            self.latent_q_rot(q, q, f, batch, heads, dim, rot_dim, rot_dims, dim)          # in place: the head's own row
            keys = torch.empty((T, heads * (dim + rot_dim)), dtype=dt, device=dev)
            self.gemm_grouped(rows, w_uk, keys, heads, T, dim, kv_rank, slot, 0, kv_rank, dim * kv_rank,
                              heads * (dim + rot_dim), dim + rot_dim)
            self._check(self.lib.tff_latent_spread(_ptr(rows), _c_int(kv_rank), _c_int(rot_dim), _ptr(keys), _c_int(dim),
                                                   _c_int(heads), _c_int(_dt(keys)), _c_int(T), self._stream()),
                        "latent_spread")
            self.launches += 1
            values = torch.empty((T, heads * vdim), dtype=dt, device=dev)
            self.gemm_grouped(rows, w_uv, values, heads, T, vdim, kv_rank, slot, 0, kv_rank, vdim * kv_rank,
                              heads * vdim, vdim)
            self.attention_tile(q, batch, block_table, kv_cache, kv_layer, page_size, out, heads, heads, dim + rot_dim,
                                vdim, scale, dense=(keys, values))
            return
        q_lat = torch.empty((T, heads * slot), dtype=dt, device=dev)
        self.gemm_grouped(q, w_uk_t, q_lat, heads, T, kv_rank, dim, heads * (dim + rot_dim), dim + rot_dim,
                          dim, kv_rank * dim, heads * slot, slot)
        self.latent_q_rot(q, q_lat, f, batch, heads, dim, rot_dim, rot_dims, kv_rank)
        o_lat = torch.empty((T, heads * kv_rank), dtype=dt, device=dev)
        self.attention_tile(q_lat, batch, block_table, kv_cache, kv_layer, page_size, o_lat, heads, 1, slot, kv_rank, scale)
        self.gemm_grouped(o_lat, w_uv, out, heads, T, vdim, kv_rank, heads * kv_rank, kv_rank, kv_rank, vdim * kv_rank,
                          heads * vdim, vdim)

    def latent_finish(self, proj, cq, q_norm_w, kv_norm_w, eps, freq, rot_dim, rot_dims, batch, block_table, kv_cache,
                      kv_layer, page_size, q_rank, kv_rank, dense_out=None) -> None:
        """csrc/latent.cu: the float32 rows [q latent | kv latent | rotated key part] -> normed query latents ``cq`` and,
        with kv_rank > 0, the token's cache slot [normed kv latent | rotated key part] (and the same vector into row t of
        ``dense_out`` [T, slot], when given)."""
        self._need_cuda(proj, cq, q_norm_w, kv_norm_w, freq, block_table)
        T = proj.shape[0]
        c_ptr, page_stride = self._layer_cache(kv_cache, kv_layer)
        clear = 1 if proj.data_ptr() in self._acc_zero else 0
        self._check(self.lib.tff_latent_finish(
            _ptr(proj), _c_int(proj.shape[1]), _c_int(clear), _c_int(q_rank), _c_int(kv_rank), _c_int(rot_dim),
            _c_int(rot_dims), _ptr(q_norm_w), _ptr(kv_norm_w), _c_float(eps), _ptr(freq), _ptr(batch.positions),
            _ptr(batch.tok_req), _ptr(block_table), _c_int(block_table.shape[1]), c_ptr if kv_rank > 0 else _vp(0),
            ctypes.c_longlong(page_stride), _c_int(page_size), _c_int(kv_cache.shape[-1]), _ptr(cq), _c_int(_dt(cq)),
            _ptr(dense_out), _c_int(T), self._stream()), "latent_finish")
        if clear:
            self._acc_zero[proj.data_ptr()] = True
        self.launches += 1

    def latent_q_rot(self, q, q_lat, freq, batch, heads, dim, rot_dim, rot_dims, kv_rank) -> None:
        """The rotated part of every query head of the rows ``q`` into its place in ``q_lat`` (same type; a head's row
        of ``q_lat`` has kv_rank + rot_dim elements, so with kv_rank = dim and q_lat = q the rotation is in place)."""
        assert q.dtype == q_lat.dtype
        self._check(self.lib.tff_latent_q_rot(_ptr(q), _c_int(dim), _c_int(rot_dim), _c_int(rot_dims), _ptr(freq),
                                              _ptr(batch.positions), _ptr(q_lat), _c_int(_dt(q_lat)), _c_int(kv_rank),
                                              _c_int(heads), _c_int(q.shape[0]), self._stream()), "latent_q_rot")
        self.launches += 1

    def rope_table(self, table, theta: float, rot_dim: int) -> None:
        """table float32 [max_pos, rot_dim/2, 2] = (cos, sin)(pos * theta^(-2i/rot_dim)).
        The frequencies exp(-(2i/d) ln theta) (src/kernel/cuda/rope_table.cu:33) are
        evaluated in double on the host and rounded once to float32."""
        self._need_cuda(table)
        half = rot_dim // 2
        assert table.dtype == torch.float32 and tuple(table.shape[1:]) == (half, 2)
        i = np.arange(half, dtype=np.float64)
        inv = np.exp(-(2.0 * i / float(rot_dim)) * math.log(theta)).astype(np.float32)
        inv_t = torch.from_numpy(inv).to(table.device)
        self._check(self.lib.tff_rope_table(_ptr(table), _ptr(inv_t), _c_int(table.shape[0]), _c_int(rot_dim),
                                            self._stream()), "rope_table")
        torch.cuda.current_stream().synchronize()   # inv_t must outlive the kernel
        self.launches += 1

    def qk_norm_rope_kv_write(self, qkv, q_out, q_w, k_w, eps, table, rot_dim, batch, block_table, kv_cache,
                              kv_layer, page_size, nq, nkv, d, write_cache) -> None:
        """qkv [T, (nq+2nkv)*d] float32 or activation type -> q_out [T, nq*d] (normed, rotated) and the
        token's K/V page slots."""
        self._need_cuda(qkv, q_out, q_w, k_w, table, block_table)
        c_ptr, _, c_layers, c_layer = self._cache_args(kv_cache, kv_layer)
        T = qkv.shape[0]
        assert qkv.shape[1] == (nq + 2 * nkv) * d and tuple(q_out.shape) == (T, nq * d)
        assert qkv.dtype in (torch.float32, q_out.dtype)
        if write_cache:
            assert kv_cache is not None and kv_cache.dtype == q_out.dtype, "cache dtype must match activations"
            assert tuple(kv_cache.shape[2:]) == (2, nkv, page_size, d)
        clear = 1 if qkv.data_ptr() in self._acc_zero else 0
        self._check(self.lib.tff_qk_norm_rope_kv_write(
            _ptr(qkv), _c_int(1 if qkv.dtype == torch.float32 else 0), _c_int(clear), _ptr(q_out), _c_int(_dt(q_out)),
            _ptr(q_w), _ptr(k_w), _c_float(eps),
            _ptr(table), _c_int(rot_dim), _c_int(table.shape[0] if table is not None else 0),
            _ptr(batch.positions), _ptr(batch.tok_req), _ptr(block_table),
            _c_int(block_table.shape[1] if block_table is not None else 0),
            c_ptr, _c_int(c_layers), _c_int(c_layer), _c_int(page_size), _c_int(1 if write_cache else 0),
            _c_int(T), _c_int(nq), _c_int(nkv), _c_int(d), self._stream()), "qk_norm_rope_kv_write")
        if clear:
            self._acc_zero[qkv.data_ptr()] = True
        self.launches += 1

    def qkv_project(self, h, w_qkv, q_out, q_w, k_w, eps, table, rot_dim, batch, block_table, kv_cache,
                    kv_layer, page_size, nq, nkv, d, write_cache) -> None:
        """The q/k/v projection of ``h`` with ``w_qkv`` ([q heads | k heads | v heads] rows), per-head RMSNorm of
        q and k, rotation, q into ``q_out`` and k, v into the tokens' cache slots.  The projection's accumulators
        stay in float32 until q and k have been normalised.  Prompt-sized bfloat16 batches with heads of 128 do all
        of it in the epilogue of the product on pairs of SMs; everything else is the product into a float32 buffer
        followed by qk_norm_rope_kv_write."""
        T, K = h.shape
        if isinstance(h, DeferredNorm):
            h = h.materialize()
        # The fused form runs on pairs of SMs only.  Where another configuration saves more waves than the separate
        # kernel costs (a pass over the float32 projection at about 5 TB/s and a launch), the projection is not fused.
        if self.USE_SM_PAIRS and T > self.SWAP_MAX_M:
            costs = self.prompt_costs(T, (nq + 2 * nkv) * d, K, False)
            apart = min(v[0] for v in costs.values()) + T * (nq + 2 * nkv) * d * 6 / 5e6 + 3.0
            pairs_pay = 512 in costs and costs[512][0] <= apart
        else:
            pairs_pay = False
        fused = (pairs_pay and d == 128 and h.dtype == torch.bfloat16
                 and w_qkv.dtype == torch.bfloat16 and q_out.dtype == torch.bfloat16 and K % 8 == 0
                 and (table is None or rot_dim == d) and (kv_cache is None or kv_cache.dtype == torch.bfloat16)
                 and (not write_cache or kv_cache is not None)
                 and all(t is None or t.data_ptr() % 16 == 0 for t in (h, w_qkv, q_out, q_w, k_w, table, kv_cache))
                 and (kv_cache is None or kv_cache.stride(0) % 8 == 0 and kv_cache.stride(1) % 8 == 0))
        if not fused:
            qkv = self.projection_buffer(T, (nq + 2 * nkv) * d, h.device, h.dtype)
            self.gemm(h, w_qkv, qkv)
            self.qk_norm_rope_kv_write(qkv, q_out, q_w, k_w, eps, table, rot_dim, batch, block_table, kv_cache,
                                       kv_layer, page_size, nq, nkv, d, write_cache)
            return
        self._need_cuda(h, w_qkv, q_out, q_w, k_w, table, block_table)
        c_ptr, _, c_layers, c_layer = self._cache_args(kv_cache, kv_layer)
        assert tuple(w_qkv.shape) == ((nq + 2 * nkv) * d, K) and tuple(q_out.shape) == (T, nq * d)
        if write_cache:
            assert tuple(kv_cache.shape[2:]) == (2, nkv, page_size, d)
        self._check(self.lib.tff_gemm_tc_qkv_rope(
            _ptr(h), _ptr(w_qkv), _c_int(T), _c_int(K), _ptr(q_out), _ptr(q_w), _ptr(k_w), _c_float(eps),
            _ptr(table), _c_int(table.shape[0] if table is not None else 0),
            _ptr(batch.positions), _ptr(batch.tok_req), _ptr(block_table),
            _c_int(block_table.shape[1] if block_table is not None else 0),
            c_ptr, _c_int(c_layers), _c_int(c_layer), _c_int(page_size), _c_int(1 if write_cache else 0),
            _c_int(nq), _c_int(nkv), self._stream()), "gemm_tc_qkv_rope")
        self.launches += 1

    def attend(self, h, w_qkv, q_w, k_w, eps, table, rot_dim, batch, block_table, kv_cache, kv_layer, page_size, out,
               nq, nkv, d, scale, window, write_cache) -> None:
        """The whole mixer between its input rows and its output projection: q/k/v projection of ``h``, per-head
        RMSNorm of q and k, rotation, cache write, attention over the paged cache -> out [T, nq*d].  How many
        kernels that is, is decided here: prompt portions with heads of 128 do everything up to the cache write in
        the projection's epilogue (qkv_project); a decode step runs projection, q/k-norm + rotation + write, and
        attention (with the merge of its key shares).  A decode attention that took the projection's float32
        accumulators and finished queries, new keys and new values itself was built and measured: one launch
        fewer and 0.05 ms a step slower at the Qwen3-8B shape (under programmatic dependent launch the small
        kernel's time already hid behind the attention's first loads of old keys), so it was not kept."""
        T = h.shape[0]
        q = torch.empty((T, nq * d), dtype=out.dtype, device=out.device)
        self.qkv_project(h, w_qkv, q, q_w, k_w, eps, table, rot_dim, batch, block_table, kv_cache, kv_layer, page_size,
                         nq, nkv, d, write_cache)
        self.attention(q, batch, block_table, kv_cache, kv_layer, page_size, out, nq, nkv, d, scale, window)

    def attention(self, q, batch, block_table, kv_cache, kv_layer, page_size, out,
                  nq, nkv, d, scale, window) -> None:
        """q [T, nq*d] (normed, rotated) against the paged cache -> out [T, nq*d]."""
        self._need_cuda(q, block_table, out)
        T = q.shape[0]
        assert kv_cache.dtype == q.dtype == out.dtype
        assert tuple(q.shape) == (T, nq * d) and tuple(out.shape) == (T, nq * d)
        assert tuple(kv_cache.shape[2:]) == (2, nkv, page_size, d)
        self._attention_dispatch(q, batch, block_table, kv_cache, kv_layer, page_size, out,
                                 nq, nkv, d, scale, window)

    def _attention_dispatch(self, q, batch, block_table, kv_cache, kv_layer, page_size, out,
                            nq, nkv, d, scale, window) -> None:
        if q.dtype == torch.bfloat16 and d in (64, 128):
            self.attention_bf16(q, batch, block_table, kv_cache, kv_layer, page_size, out, nq, nkv, d, scale, window)
        else:
            self.attention_generic(q, batch, block_table, kv_cache, kv_layer, page_size, out, nq, nkv, d, scale, window)

    def attention_splits(self, num_requests: float, max_q_len: int, nq: int, nkv: int) -> int:
        """Shares of the key range per tile, for ``num_requests`` requests of one context length (for
        unequal contexts: sum / longest, effective_requests above).  The count is rounded to a
        power of two, so that a step replayed as a CUDA graph, captured for such a class, and an eager
        step cut alike."""
        if max_q_len * (nq // nkv) > 16:
            return 1                                   # portions: enough tiles already
        b = nearest_power_of_two(num_requests)
        # One wave of two CTAs per SM.  With more work items than that the grid runs in rounds and the last one is
        # seldom full (64 requests of 8 heads on 296 slots: two rounds for 1.73 rounds' worth of work); cutting
        # the items so that the rounds fill was measured and lost (4 shares: 7.36 against 6.76 ms a step at 64
        # requests): every share pays its own ramp, and the partial results another pass.
        return max(1, min(16, 2 * self.NUM_SMS // (b * nkv)))

    MIXED_SHARES_FROM = 6144      # keys behind a small portion from which it is cut into shares beside decoded tokens too

    def portion_splits(self, num_requests: int, max_q_len: int, max_kv_len: int, nq: int, nkv: int) -> int:
        """Shares of the key range for a step that is prompt portions only.  A portion of few tokens behind a long
        context (the last piece of a prompt, what a step's token budget left over) is one or two tiles a key/value
        head: as tensor-core tiles of 128 rows they walk the whole context on 8 or 16 SMs.  Up to 256 packed rows
        (tokens times query heads a key/value head) behind 2,048 keys or more, such portions go to the kernel of
        64-row tiles with the key range cut into shares, as many as give every SM two CTAs.  A whole step of the
        8B shape with 16 tokens behind 4,000: 7.2 -> 5.1 ms; behind 16,000: 16.1 -> 6.8; 64 behind 16,000: 14.5 ->
        10.1; behind 1,000 keys it loses (5.4 -> 5.6), and above 256 rows the tensor-core kernel is the faster one
        (96 tokens behind 2,048: 60 against 65 us a layer)."""
        rows = max_q_len * (nq // nkv)
        if rows <= 16 or rows > 256 or max_kv_len < 2048:
            return 1
        ctas = -(-rows // 64) * nkv * max(1, num_requests)
        blocks = -(-max_kv_len // 64)
        s = 1
        while s < 16 and ctas * s * 2 <= 2 * self.NUM_SMS and s * 2 <= blocks:
            s *= 2
        return s

    @staticmethod
    def key_split_class(kv_lens) -> int:
        """The class of a batch of decoded tokens that fixes how their key ranges are shared out: a step
        replayed as a CUDA graph is captured per class."""
        return nearest_power_of_two(effective_requests(kv_lens))

    def _side_stream(self, device):
        """The second stream (and the two events to fork to it and join from it), made at first use."""
        if getattr(self, "_side", None) is None:
            self._side = torch.cuda.Stream(device=device)
            self._fork, self._join = torch.cuda.Event(), torch.cuda.Event()
        return self._side

    def _decode_splits(self, batch, first: int, count: int, max_q_len: int, nq: int, nkv: int) -> int:
        """The key split for requests [first, first + count) in the order of ``batch.req_order``."""
        if batch.key_split_class is not None:
            eff = batch.key_split_class
        elif batch.h_sorted_kv_lens is not None:
            eff = effective_requests(batch.h_sorted_kv_lens[first:first + count])
        else:
            eff = count
        return self.attention_splits(eff, max_q_len, nq, nkv)

    def attention_bf16(self, q, batch, block_table, kv_cache, kv_layer, page_size, out,
                       nq, nkv, d, scale, window, num_splits=None, extra=(0.0, False, None)) -> None:
        """Flash attention over the paged cache (head sizes 64 and 128).  Requests that bring so few
        tokens that they fit a 16-row tile (decoded tokens) and requests that bring long portions are
        launched apart when a step holds both, each with the kernel made for it.  ``extra`` = (softcap, sink,
        gates): a cap on the scores, a sink in the softmax, a float32 [T, nq] multiplier of the heads' outputs."""
        G = nq // nkv
        sq = batch.h_sorted_q_lens
        B = batch.num_requests
        n_short = int(np.searchsorted(sq, 16 // G, side="right")) if (sq is not None and num_splits is None) else 0
        if 0 < n_short < B and batch.req_order is not None:
            # The two launches write different rows of ``out`` and read what the kernels before them wrote:
            # they run side by side, the decoded tokens' on a second stream.  The portions' kernel is
            # launched first; it seldom fills the SMs (a 512-token portion is 80 to 160 CTAs of one an SM),
            # and the other one, bound by memory, runs on what is left.
            main = torch.cuda.current_stream()
            side = None if torch.cuda.is_current_stream_capturing() else self._side_stream(q.device)
            if side is not None:
                self._fork.record(main)
            # (One share for the portions here unless their context is long: their few CTAs run beside the decoded
            # tokens' kernel, which has the other SMs; cut into shares they contend with it for all of them.  Measured:
            # the 14B mixed workload, contexts up to 4,096, 3.52-3.61 s with shares against 3.35-3.37 without; a step of
            # the 8B shape with 16 tokens behind 4,000 keys beside 8 decoded tokens 8.2 against 8.1 ms, behind 8,000 keys
            # 8.1 against 10.6, behind 16,000 keys 8.1 against 15.9.)
            long_kv = int(batch.h_sorted_kv_lens[n_short:].max()) if batch.h_sorted_kv_lens is not None else 0
            shares = self.portion_splits(B - n_short, int(sq[-1]), long_kv, nq, nkv) if long_kv >= self.MIXED_SHARES_FROM else 1
            self._attention_bf16_launch(q, batch, block_table, kv_cache, kv_layer, page_size, out, nq, nkv, d, scale,
                                        window, shares, batch.req_order[n_short:], B - n_short, int(sq[-1]), extra)
            splits = self._decode_splits(batch, 0, n_short, int(sq[n_short - 1]), nq, nkv)
            if side is None:
                self._attention_bf16_launch(q, batch, block_table, kv_cache, kv_layer, page_size, out, nq, nkv, d,
                                            scale, window, splits, batch.req_order[:n_short], n_short,
                                            int(sq[n_short - 1]), extra)
            else:
                side.wait_event(self._fork)
                with torch.cuda.stream(side):
                    self._attention_bf16_launch(q, batch, block_table, kv_cache, kv_layer, page_size, out, nq, nkv,
                                                d, scale, window, splits, batch.req_order[:n_short], n_short,
                                                int(sq[n_short - 1]), extra)
                    self._join.record(side)
                main.wait_event(self._join)
        else:
            if num_splits is None:
                if batch.max_q_len * G > 16:
                    num_splits = self.portion_splits(B, batch.max_q_len, batch.max_kv_len, nq, nkv)
                else:
                    num_splits = self._decode_splits(batch, 0, B, batch.max_q_len, nq, nkv)
            # decoded tokens only: longest contexts first (the order the batch was packed with)
            order = batch.req_order if n_short == B else None
            self._attention_bf16_launch(q, batch, block_table, kv_cache, kv_layer, page_size, out, nq, nkv, d, scale,
                                        window, num_splits, order, B, batch.max_q_len, extra)

    def _attention_bf16_launch(self, q, batch, block_table, kv_cache, kv_layer, page_size, out, nq, nkv, d, scale,
                               window, num_splits, req_ids, num_requests, max_q_len, extra=(0.0, False, None)) -> None:
        T = q.shape[0]
        splits = num_splits
        c_ptr, c_pages, c_layers, c_layer = self._cache_args(kv_cache, kv_layer)
        ws = None
        if splits > 1:
            need = T * nq * splits * (d + 2)
            if max_q_len * (nq // nkv) > 16:
                # portions cut into shares: one buffer that only grows, since their sizes change from step to step and
                # a fresh size may cost an allocation from the driver in the middle of serving
                ws = getattr(self, "_portion_ws", None)
                if ws is None or ws.numel() < need or ws.device != q.device:
                    ws = torch.empty(max(need, 1 << 22), dtype=torch.float32, device=q.device)
                    self._portion_ws = ws
            else:
                ws = torch.empty(need, dtype=torch.float32, device=q.device)
        softcap, sink, gates = extra
        sink_on, sink_val = self._sink_args(sink, nq)
        self._check(self.lib.tff_attention_bf16_paged_ext(
            _ptr(q), _ptr(batch.q_start), _ptr(batch.pos_start), _ptr(req_ids), _ptr(block_table),
            _c_int(block_table.shape[1]),
            c_ptr, ctypes.c_longlong(c_pages), _c_int(c_layers), _c_int(c_layer),
            _c_int(page_size),
            _ptr(out), _ptr(ws), _c_int(T), _c_int(num_requests), _c_int(max_q_len), _c_int(splits),
            _c_int(nq), _c_int(nkv), _c_int(d), _c_float(scale), _c_int(window), _c_float(softcap),
            _c_int(1 if sink_on else 0), _ptr(sink_val), _ptr(gates), self._stream()), "attention_bf16")
        self.launches += 2 if splits > 1 else 1

    def attention_generic(self, q, batch, block_table, kv_cache, kv_layer, page_size, out,
                          nq, nkv, d, scale, window) -> None:
        T = q.shape[0]
        c_ptr, _, c_layers, c_layer = self._cache_args(kv_cache, kv_layer)
        self._check(self.lib.tff_attention_generic(
            _ptr(q), _c_int(_dt(q)), _c_int(q.shape[1]),
            _ptr(batch.positions), _ptr(batch.tok_req), _ptr(block_table), _c_int(block_table.shape[1]),
            c_ptr, _c_int(c_layers), _c_int(c_layer), _c_int(page_size),
            _ptr(out), _c_int(T), _c_int(nq), _c_int(nkv), _c_int(d), _c_float(scale), _c_int(window),
            self._stream()), "attention_generic")
        self.launches += 1

    def gemm_swiglu(self, a, w_gate_up, out) -> None:
        """out[T, I] = silu(a @ Wg^T) * (a @ Wu^T), w_gate_up being merge_gate_up(Wg, Wu)."""
        self.gemm_gated_act(a, w_gate_up, out, "silu")

    def gemm_gated_act(self, a, w_gate_up, out, activation: str) -> None:
        """out[T, I] = act(a @ Wg^T) * (a @ Wu^T), act "silu" or "gelu_tanh"."""
        self._need_cuda(a, w_gate_up, out)
        T, I = out.shape
        K = a.shape[1]
        block = self.gate_up_block(I)
        tc = (a.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16 and K % 8 == 0
              and a.data_ptr() % 16 == 0 and w_gate_up.data_ptr() % 16 == 0)
        if tc and T > self.CLUSTER_MAX_M and block == 64 and out.dtype == torch.bfloat16 and out.data_ptr() % 16 == 0:
            # the activation is applied in the product's epilogue, in the normal orientation from 17 rows on: the
            # swapped product and the SwiGLU kernel behind it took 45 us at 72 rows of the 8B shape against 39, 78
            # against 59 at 256
            bn = self.prompt_plan(T, 2 * I, K, False)[1]
            self._check(self.lib.tff_gemm_tc_gated(_ptr(a), _ptr(w_gate_up), _ptr(out), _c_int(T), _c_int(I),
                                                   _c_int(K), _c_int(bn), _c_int(self.ACTIVATION_CODES[activation]),
                                                   self._stream()), "gemm_tc_gated")
            self.launches += 1
            return
        small = tc and T <= self.SWAP_MAX_M
        if small:
            gu = self.projection_buffer(T, 2 * I, out.device, out.dtype, use="act")
        else:
            gu = torch.empty((T, 2 * I), dtype=out.dtype, device=out.device)
        self.gemm(a, w_gate_up, gu)
        self.gated_act(gu, out, block, activation)

    def argmax(self, logits, out) -> None:
        self._need_cuda(logits, out)
        R, V = logits.shape
        assert logits.dtype == torch.float32 and out.dtype == torch.int32 and out.numel() == R
        scratch = getattr(self, "_argmax_scratch", None)
        if scratch is None or scratch.device != logits.device:
            # 64 ticket counters (kept at zero by the kernel), then the candidates of 16 shares for up to 64 rows
            scratch = torch.zeros(64 + 2 * 64 * 16, dtype=torch.int32, device=logits.device)
            self._argmax_scratch = scratch
        use = scratch
        self._check(self.lib.tff_argmax(_ptr(logits), _ptr(out), _c_int(R), _c_int(V), _ptr(use), self._stream()), "argmax")
        self.launches += 1

    def sample(self, logits, temperature, uniform, out, top_k=None, top_p=None, min_p=None) -> None:
        self._need_cuda(logits, temperature, uniform, out, top_k, top_p, min_p)
        R, V = logits.shape
        assert logits.dtype == torch.float32 and out.dtype == torch.int32
        assert temperature.dtype == torch.float32 and uniform.dtype == torch.float32
        self._check(self.lib.tff_sample(_ptr(logits), _ptr(temperature), _ptr(uniform), _ptr(top_k), _ptr(top_p),
                                        _ptr(min_p), _ptr(out), _c_int(R), _c_int(V), self._stream()), "sample")
        self.launches += 1

    def repetition_penalty(self, logits, rows, tokens, penalty) -> None:
        self._need_cuda(logits, rows, tokens, penalty)
        n = rows.numel()
        assert logits.dtype == torch.float32 and rows.dtype == torch.int32 and tokens.dtype == torch.int32
        assert penalty.dtype == torch.float32 and tokens.numel() == n and penalty.numel() == n
        self._check(self.lib.tff_repetition_penalty(_ptr(logits), _ptr(rows), _ptr(tokens), _ptr(penalty),
                                                    _c_int(n), _c_int(logits.shape[1]), self._stream()),
                    "repetition_penalty")
        self.launches += 1
