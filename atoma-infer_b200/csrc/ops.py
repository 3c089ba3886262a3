"""The kernels as Python calls on torch tensors.

Every function launches hand-written CUDA from the libraries under ``kernels/``
on torch's current stream; tensors are only memory here.  There is no CPU path:
without a CUDA device the constructor raises.  Matrix products of the bfloat16
path with many rows go to cuBLAS through ``torch.mm``, as the reference sends
its linears to cuBLAS through candle (models/src/llama.rs:269-271); the gate/up
product of long prompts, with its activation, runs on the tcgen05 kernel here.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from . import build

DT_F32, DT_BF16 = 0, 1
META_HEADER_INTS = 20
META_NUM_TOKENS, META_NUM_ENTRIES, META_NUM_ROWS, META_BT_STRIDE, META_BT_OFFSET = 0, 1, 2, 4, 12
MAX_GROUPS = 8
STATUS_WORDS = 8
SKINNY_MAX_ROWS = 16  # bfloat16 linears with at most this many rows stream the weights

CORE_SOURCES = ["kernels/core.cu", "kernels/layer_ops.cu", "kernels/linear_bf16.cu", "kernels/linear_stream.cu", "kernels/sampling.cu"]
ATTENTION_SOURCES = ["kernels/attention_bf16.cu"]
GEMM_SOURCES = ["kernels/gemm_tcgen05.cu"]
ATTENTION_TC_SOURCES = ["kernels/attention_tcgen05.cu"]
DECODE_STACK_SOURCES = ["kernels/decode_stack.cu"]
# parallel blocks, state-space mixers, latent attention, routed experts: built when a model first uses one of them
MIXER_SOURCES = ["kernels/stream_ops.cu", "kernels/ssm.cu", "kernels/latent.cu", "kernels/moe.cu", "kernels/gated_stream.cu"]
# recurrences whose decay differs from row to row (gated linear attention, the selective scan): built at first use too
RECURRENT_SOURCES = ["kernels/recurrent.cu"]
ATTENTION_TC_HEAD_DIMS = (64, 128)  # head sizes of the tcgen05 prefill attention
ATTENTION_HEAD_DIMS = tuple(range(16, 257, 16))  # every head size the kernels take; the build check builds them all, a model only its own


class KernelError(RuntimeError):
    pass


def _code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return DT_F32
    if t.dtype == torch.bfloat16:
        return DT_BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {t.dtype}")


def _p(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)


class CudaOps:
    """Loads (building at first use) the kernel library and exposes its entry points."""

    def __init__(self, device: torch.device):
        if not torch.cuda.is_available():
            raise KernelError("this engine runs on a CUDA device only; none is available")
        self.device = torch.device(device)
        self.lib = build.load_library("core", CORE_SOURCES, cuda=True)
        self.status = torch.zeros(STATUS_WORDS, dtype=torch.int32, device=self.device)
        self.launches = 0  # own kernel launches, counted for the benchmark record
        self._attn_libs = {}
        self._attn_tc_libs = {}
        # levers for the kernel tests (each kernel is compared with the one it stands in for)
        self.tc_attention = True    # tcgen05 prefill attention where the geometry allows
        self.decode_cluster = True  # split merge of the decode attention inside a cluster
        self.tc_gemm = True         # gate/up + SwiGLU of long prompts on tcgen05
        # large decode batches: key tiles dealt out evenly over as many blocks as the GPU holds ("0": never;
        # a number above 1: always, with that many blocks, for experiments and tests)
        flat = os.environ.get("ATOMA_INFER_DECODE_FLAT", "1")
        self.decode_flat = flat != "0"
        self.decode_flat_forced = int(flat) if flat.isdigit() and int(flat) > 1 else 0
        self._flat_blocks = {}
        self._gemm_lib = None
        self.last_tokens = torch.zeros(1 << 16, dtype=torch.int32, device=self.device)  # by state slot
        self._counters = torch.zeros(1 << 16, dtype=torch.int32, device=self.device)  # split arrivals; kernels leave zeros
        # Programmatic dependent launch lets a kernel start while its predecessor drains (its weight
        # loads are in flight before the dependency wait).  Blocks that have started early wait for the
        # kernel before them and slow it down while they do, so only kernels whose wait is short start
        # early: the few-row linears and the decode attention release their dependents when they start
        # themselves; the norm kernel, which also starts early, releases its dependents only once its own
        # wait is over (else the linear after it would wait through the whole linear before it).  Measured
        # on the decode step of Llama 3.2 1B: off 0.967 ms; linears and attention 0.918 ms; with the norm
        # 0.906 ms; every kernel, each releasing its dependents at once, 1.17 ms.
        # ATOMA_INFER_PDL: "0" off, "1" every kernel, "linear" without the norm, default "linear+norm".
        mode = os.environ.get("ATOMA_INFER_PDL", "linear+norm")
        self.pdl = {"0": 0, "1": 1, "linear": 2, "linear+norm": 6}.get(mode, 6)
        self.fused_rope = True  # the decode attention rotates q and k and writes the new key and value itself
        self.masked_fast_attention = True  # chunk masks and sinks on the tensor-core attention kernels (False: on the plain one; a test lever)
        self.scored_fast_attention = True  # likewise score caps, distance slopes and windows that keep the first tokens
        # Few-row linears go to the persistent, TMA-fed kernel (kernels/linear_stream.cu) where it is the faster one
        # (see _stream_linear); ATOMA_INFER_STREAM_LINEAR=0 keeps them all on the kernel that loads weights into
        # fragments directly (kernels/linear_bf16.cu).  The kernel tests set the attribute.
        self.stream_linear = os.environ.get("ATOMA_INFER_STREAM_LINEAR", "1") != "0"
        self.stream_min_rows = int(os.environ.get("ATOMA_INFER_STREAM_MIN_ROWS", "1"))  # a test and measurement lever
        # In decode steps whose linears are streamed, the RMSNorms between them are folded into them (parts/decode_stack.py,
        # the chain); ATOMA_INFER_FOLD_NORMS=0 leaves the norm a kernel of its own.
        self.fold_norms = os.environ.get("ATOMA_INFER_FOLD_NORMS", "1") != "0"
        # Decode steps of at most 16 rows can run stretches of whole layers as one persistent kernel (ATOMA_INFER_FUSED_LAYERS=1;
        # off by default while it is slower than the step part by part)
        self.fused_layers = os.environ.get("ATOMA_INFER_FUSED_LAYERS", "0") == "1"
        self._stack_libs, self._stack_blocks = {}, {}
        # Before the decode attention of a small batch the weight of the linear after it is asked into L2 if it has
        # at most this many bytes (0: never); see _prefetch_next_weight.
        self.prefetch_bytes = int(float(os.environ.get("ATOMA_INFER_PREFETCH_MB", "12")) * (1 << 20))
        self._order, self._order_index, self._starts, self._cursor = [], {}, [], 0
        # ... on a stream of its own when the step has at most this many rows, else as a link of the step's chain
        self.prefetch_aside_rows = int(os.environ.get("ATOMA_INFER_PREFETCH_ASIDE_ROWS", "4"))
        self._side_stream, self._side_pending = None, False
        self.lib.kernels_set_pdl(int(self.pdl))
        self.num_sms = torch.cuda.get_device_properties(self.device).multi_processor_count

    # ------------------------------------------------------------------ helpers
    def _stream(self):
        return ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def _check(self, err: int, what: str):
        self.launches += 1
        if err:
            raise KernelError(f"{what}: CUDA error {err}")

    def set_pdl(self, on: bool) -> None:
        self.pdl = int(on)
        self.lib.kernels_set_pdl(int(on))
        for lib in self._attn_libs.values():
            lib.kernels_set_pdl(1 if on else 0)
        for name in ("_mixer_lib", "_recurrent_lib"):
            if getattr(self, name, None) is not None:
                getattr(self, name).kernels_set_pdl(int(on))

    @staticmethod
    def describe_status(words) -> Optional[str]:
        """What the status words say (None: nothing).  Kernels write them instead of trapping or hanging."""
        s = list(words)
        if not any(s):
            return None
        return (f"token id out of range at token {s[0] - 1}" if s[0] else
                f"block table names no valid page for token {s[1] - 1}" if s[1] else
                f"a tensor-core GEMM block ({s[2] - 1}) gave up waiting on a barrier" if s[2] else
                f"a tensor-core attention block ({s[3] - 1}) gave up waiting on a barrier" if s[3] else
                f"a block ({s[4] - 1}) of the decode step's layer kernel gave up waiting" if s[4] else
                f"a block ({s[5] - 1}) of the streamed few-row linear gave up waiting" if s[5] else
                f"status words {s}")

    def clear_status(self) -> None:
        self.status.zero_()

    def check_status(self) -> None:
        """Raises if a kernel of an earlier launch met a bad token id or page id, or gave up a wait
        (synchronises)."""
        what = self.describe_status(self.status.tolist())
        if what:
            self.clear_status()
            raise KernelError("device status: " + what)

    # ------------------------------------------------------------------ weights ahead of time
    def set_weight_order(self, weights) -> None:
        """The weight matrices of the model's linears in the order a step streams them (a model tells this once,
        after binding)."""
        self._order = [(w.data_ptr(), w.numel() * w.element_size()) for w in weights]
        self._starts, at = [], 0
        for _, n in self._order:
            self._starts.append(at)
            at += n
        self._order_index = {}
        for i, (ptr, _) in enumerate(self._order):
            self._order_index.setdefault(ptr, []).append(i)
        self._cursor = 0

    def _note_weight(self, w) -> None:
        where = self._order_index.get(w.data_ptr())
        if where:
            self._cursor = next((k for k in where if k >= self._cursor), where[0]) + 1

    def _prefetch_next_weight(self, rows: int = 0) -> None:
        """Before the decode attention of a small batch: asks the weight of the linear after it (the next one in the
        stream after the last linear that ran) into L2, if it is a small one (``prefetch_bytes`` at most).  A small
        matrix is read in a few microseconds that are mostly start-up and drain; read from L2 it is shorter, and the
        attention of a small batch leaves the bandwidth to bring it there.  Measured, decode step at batch 8: Llama
        3.2 1B (8.4 MB) 0.924 -> 0.897 ms; asking for more than that one weight, or from inside the linears, is
        slower; at the 3B and 8B sizes (18.9 and 33.5 MB) asking at all is 3 to 5 % slower, hence the limit.
        ``rows``: the step's rows.  With at most ``prefetch_aside_rows`` of them (ATOMA_INFER_PREFETCH_ASIDE_ROWS) the
        request runs on a stream of its own beside the step's chain; measured in the chain against beside it, decode
        step of Llama 3.2 1B: batch 1 0.744 / 0.730 ms, batch 2 0.763 / 0.744, batch 4 0.773 / 0.745, batch 8 0.820 /
        0.839."""
        if self._cursor >= len(self._order):
            return
        ptr, size = self._order[self._cursor]
        if size > self.prefetch_bytes:
            return
        if rows > self.prefetch_aside_rows:
            self._check(self.lib.l2_prefetch(1, (ctypes.c_void_p * 1)(ptr), (ctypes.c_ulonglong * 1)(size), self._stream()),
                        "l2_prefetch")
            return
        # on a stream of its own, after what the step has launched so far: the attention then follows the projection
        # directly in the chain of dependent launches
        main = torch.cuda.current_stream(self.device)
        if self._side_stream is None:
            self._side_stream = torch.cuda.Stream(self.device)
        fork = torch.cuda.Event()
        fork.record(main)
        self._side_stream.wait_event(fork)
        self._check(self.lib.l2_prefetch_aside(1, (ctypes.c_void_p * 1)(ptr), (ctypes.c_ulonglong * 1)(size),
                                               ctypes.c_void_p(self._side_stream.cuda_stream)), "l2_prefetch")
        self._side_pending = True

    def join_side_work(self) -> None:
        """What ran beside the step's stream (see _prefetch_next_weight) joins it: called at the end of a forward pass."""
        if self._side_pending:
            done = torch.cuda.Event()
            done.record(self._side_stream)
            torch.cuda.current_stream(self.device).wait_event(done)
            self._side_pending = False

    # ------------------------------------------------------------------ kernels
    def embed(self, tokens, table, resid, meta, T: int, scale: float = 1.0):
        """resid[t] = scale * table[tokens[t]].  A token id -1 - s means: the token last sampled into slot s
        (``self.last_tokens``)."""
        H, V = table.shape[1], table.shape[0]
        self._check(self.lib.embed_rows(_p(tokens), _p(table), _code(table), _p(resid), _p(meta), T, H, V,
                                        ctypes.c_float(scale), _p(self.last_tokens), self.last_tokens.numel(),
                                        _p(self.status), self._stream()), "embed_rows")

    def add_rmsnorm(self, resid, delta, w, eps: float, out, meta, n: int, rows=None):
        """resid += delta (if given); out = rmsnorm(resid) * w.  With ``rows`` the sum and the
        norm are taken at those rows only and resid is left as it is."""
        H = resid.shape[-1]
        self._check(self.lib.add_rmsnorm(_p(resid), _p(delta), _code(delta) if delta is not None else _code(out),
                                         _p(rows), _p(w), ctypes.c_float(eps), _p(out), _code(out), _p(meta), n, H,
                                         self._stream()), "add_rmsnorm")

    def linear(self, x, w, *, out_dtype=None, silu_mul: bool = False, meta=None, use_rows: bool = False):
        """x [M, K] times w [N, K] transposed.  ``silu_mul``: w is [gate; up] stacked and the
        result is silu(gate part) * (up part), of N/2 columns."""
        M, K = x.shape
        N = w.shape[0]
        out_dtype = out_dtype or x.dtype
        n_out = N // 2 if silu_mul else N
        if x.dtype == torch.float32:
            y = torch.empty((M, N), dtype=torch.float32, device=x.device)
            self._check(self.lib.gemm_f32(_p(x), _p(w), _p(y), M, N, K, self._stream()), "gemm_f32")
            if silu_mul:
                out = torch.empty((M, n_out), dtype=torch.float32, device=x.device)
                self.silu_mul(y, out, meta, M, n_out)
                return out
            return y
        if self._stream_linear(M, N, K) and x.is_contiguous() and w.is_contiguous():
            return self.linear_streamed(x, w, out_dtype=out_dtype, silu_mul=silu_mul)
        if M <= SKINNY_MAX_ROWS and K % 8 == 0:
            y = torch.empty((M, n_out), dtype=out_dtype, device=x.device)
            self._note_weight(w)
            self._check(self.lib.linear_skinny(_p(x), _p(w), _p(y), _code(y), int(silu_mul), _p(meta), int(use_rows),
                                               M, N, K, self._stream()), "linear_skinny")
            return y
        if silu_mul and out_dtype == x.dtype and self._swiglu_on_tcgen05(M, n_out, K):
            return self.gemm_tc(x, w, silu_mul=True, bn=256)
        if out_dtype == torch.float32:
            y = torch.mm(x, w.t(), out_dtype=torch.float32)
        else:
            y = torch.mm(x, w.t())
        if silu_mul:
            out = torch.empty((M, n_out), dtype=x.dtype, device=x.device)
            self.silu_mul(y, out, meta, M, n_out)
            return out
        return y

    def linear_streamed(self, x, w, *, out_dtype=None, silu_mul: bool = False, scale_from=None, add_into=None):
        """``linear`` on the TMA-fed persistent kernel whatever the policy says (bfloat16, at most 16 rows, K a multiple
        of 64, contiguous operands).  An RMSNorm can be folded into the linears around it:
        ``add_into=(resid, next_w)``: the linear before a norm.  Nothing is returned as y; the product is added into the
        float32 residual and, with ``next_w`` (the norm's weight; None if no norm follows), the call returns
        ``(xw, ss)``: the new residual times that weight in bfloat16, and per 16-column tile and row the sum of squares.
        ``scale_from=(ss, width, eps)``: the linear after the norm, given ``xw`` as x: its rows are scaled by 1 / rms."""
        M, K = x.shape
        N = w.shape[0]
        self._note_weight(w)
        ss_in, parts, width, eps = (None, 0, 0, 0.0) if scale_from is None else (scale_from[0], scale_from[0].numel() // 16,
                                                                                 scale_from[1], scale_from[2])
        if add_into is not None:
            resid, next_w = add_into
            xw = torch.empty((M, N), dtype=torch.bfloat16, device=x.device) if next_w is not None else None
            ss = torch.empty(-(-N // 16) * 16, dtype=torch.float32, device=x.device) if next_w is not None else None
            self._check(self.lib.linear_stream_norm(_p(x), _p(w), None, DT_BF16, 2, M, N, K, _p(ss_in), parts, width,
                                                    ctypes.c_float(eps), _p(resid), _p(next_w), _p(xw), _p(ss), _p(self.status),
                                                    self._stream()), "linear_stream_norm")
            return xw, ss
        y = torch.empty((M, N // 2 if silu_mul else N), dtype=out_dtype or x.dtype, device=x.device)
        self._check(self.lib.linear_stream_norm(_p(x), _p(w), _p(y), _code(y), int(silu_mul), M, N, K, _p(ss_in), parts, width,
                                                ctypes.c_float(eps), None, None, None, None, _p(self.status), self._stream()),
                    "linear_stream_norm")
        return y

    def _stream_linear(self, M: int, N: int, K: int) -> bool:
        """Whether a bfloat16 linear of M <= 16 rows runs on the TMA-fed persistent kernel: whenever it can (K a multiple
        of 64).  Measured, decode step as a CUDA graph, all linears direct against all streamed: Llama 3.2 1B sizes, batch
        1 / 2 / 4 / 8 / 12 / 16: 0.758 / 0.800 / 0.831 / 0.878 / 1.125 / 1.265 ms against 0.778 / 0.791 / 0.805 / 0.829 /
        0.918 / 0.944, and with the norms folded into the streamed linears (up to 8 rows) 0.746 / 0.763 / - / 0.826;
        8 layers of the 3B sizes, batch 1 / 8: 0.539 / 0.656 against 0.535 (folded) / 0.641; of the 8B sizes: 0.918 / 1.040
        against 0.802 / 0.912.  The direct kernel is a quarter to a third slower with two n-tiles (9 to 16 rows).  Mixing
        the two within a layer is the slowest choice (3B sizes, batch 8: streamed only where its tiles fill the blocks
        evenly 0.733 to 0.751 ms; 1B sizes, batch 1, gate/up alone streamed 0.837): a persistent kernel holds every
        multiprocessor's shared memory until its blocks leave, so a kernel of another kind after it cannot start early.
        ``stream_min_rows`` (ATOMA_INFER_STREAM_MIN_ROWS) keeps steps of fewer rows on the direct kernel."""
        if not self.stream_linear or M > SKINNY_MAX_ROWS or K % 64:
            return False
        return M >= self.stream_min_rows

    def _swiglu_on_tcgen05(self, M: int, n_out: int, K: int) -> bool:
        """Whether the gate/up product with the SwiGLU epilogue runs on the persistent tcgen05 kernel instead
        of the library product followed by the activation kernel.  It wins when its 128 x 128 output tiles
        fill whole rounds of the multiprocessors (measured at hidden 2048, intermediate 8192: 104 against
        112 us at 2,048 rows, 198 against 213 us at 4,096; a tie at 1,536; slower below and at 3,000)."""
        if not self.tc_gemm or M < 1536 or K % 8 or n_out % 8:
            return False
        tiles = -(-M // 128) * -(-n_out // 128)
        rounds = -(-tiles // self.num_sms)
        return tiles >= 0.97 * rounds * self.num_sms

    def gemm_tc(self, a, b, *, out_dtype=None, silu_mul: bool = False, transpose: bool = False, bn: int = 256,
                ksplit: int = 1, persistent: bool = True, out=None):
        """C = A * B^T on tcgen05/TMEM with TMA-fed tiles (kernels/gemm_tcgen05.cu).  a [RA, K] fills the
        128-row side of the MMA, b [RB, K] the BN-column side.  ``transpose``: the result is [RB, RA]
        (used with a = weights when the activations have few rows).  ``silu_mul``: b is [gate; up]
        stacked and the result has RB/2 columns.  ``ksplit``: blocks of a cluster that share a tile's K.
        ``persistent`` (untransposed, unsplit): one block per multiprocessor walks the tiles and stores a tile
        while the tensor core computes the next."""
        if self._gemm_lib is None:
            self._gemm_lib = build.load_library("gemm_tcgen05", GEMM_SOURCES, cuda=True)
        out_dtype = out_dtype or a.dtype
        ra, K = a.shape
        rb = b.shape[0] // 2 if silu_mul else b.shape[0]
        shape = (rb, ra) if transpose else (ra, rb)
        c = out if out is not None else torch.empty(shape, dtype=out_dtype, device=a.device)
        self._check(self._gemm_lib.gemm_tcgen05(_p(a), _p(b), _p(c), ra, rb, K, shape[1], _code(c), int(silu_mul),
                                                int(transpose), bn, ksplit, int(persistent and not transpose and ksplit == 1),
                                                _p(self.status), self._stream()),
                    "gemm_tcgen05")
        return c

    def silu_mul(self, gu, out, meta, T: int, inter: int):
        self._check(self.lib.silu_mul(_p(gu), _p(out), _code(gu), _p(meta), T, inter, self._stream()), "silu_mul")

    # ------------------------------------------------------------------ layers other than the plain pre-norm block
    @staticmethod
    def _slot_stride(state) -> ctypes.c_longlong:
        """Floats from one slot's ring to the next (a part's state is a slice of the layer's per-request state)."""
        if state is None:
            return ctypes.c_longlong(0)
        if state.dtype != torch.float32 or state.dim() != 3 or state[0].stride() != (state.shape[2], 1):
            raise KernelError("a convolution state is float32 [slots, rows, channels] with contiguous rows")
        return ctypes.c_longlong(state.stride(0))

    def short_conv(self, x, w, state, ctx, out, *, add_input: bool = True):
        """out[t] = (x[t] +) sum_j w[j] * x[t - taps + 1 + j] over the float32 residual rows of each request, zeros
        before its start; ``w`` is float32 [taps, C]; rows before the step's portion come from ``state`` (float32
        [slots, taps - 1, C], the row of position p at place p mod (taps - 1); None when taps is 1).
        ``short_conv_save`` writes the state afterwards."""
        taps, C = w.shape
        self._check(self.lib.short_conv(_p(x), _p(w), _p(state), _p(out), _code(out), _p(ctx.meta), _p(ctx.positions),
                                        _p(ctx.token_entry), _p(ctx.cu_tokens), _p(ctx.state_slots), ctx.T, C, taps,
                                        int(add_input), self._slot_stride(state), self._stream()), "short_conv")

    def short_conv_save(self, x, state, ctx, taps: int):
        """The last taps - 1 rows of x of every entry go to its state (see ``short_conv``)."""
        if taps > 1:
            self._check(self.lib.short_conv_save(_p(x), _p(state), _p(ctx.meta), _p(ctx.positions), _p(ctx.token_entry),
                                                 _p(ctx.cu_tokens), _p(ctx.state_slots), ctx.T, x.shape[1], taps,
                                                 self._slot_stride(state), self._stream()), "short_conv_save")

    def scaled_add_rmsnorm(self, resid, delta, alpha: float, w, eps: float, ctx, *, keep=None, conv=None):
        """The norm after the sum: resid <- rmsnorm(alpha * resid + delta) * w, in place, float32.
        ``keep=(state, taps)``: the rows as they were before go to that convolution state (the last taps - 1 of every
        entry).  ``conv=(w [taps, H], state, out)``, decode steps only: also out <- new row + short convolution of it
        over ``state``, the input of the sublayer that follows."""
        H = resid.shape[1]
        k_state, k_taps = keep if keep is not None else (None, 0)
        c_w, c_state, c_out = conv if conv is not None else (None, None, None)
        self._check(self.lib.scaled_add_rmsnorm(_p(resid), _p(delta), _code(delta) if delta is not None else DT_F32,
                                                ctypes.c_float(alpha), _p(w), ctypes.c_float(eps), _p(ctx.meta), ctx.T, H,
                                                _p(k_state), int(k_taps), self._slot_stride(k_state), self._slot_stride(c_state),
                                                _p(ctx.positions), _p(ctx.token_entry),
                                                _p(ctx.cu_tokens), _p(ctx.state_slots), _p(c_w), _p(c_state),
                                                c_w.shape[0] if c_w is not None else 0, _p(c_out),
                                                _code(c_out) if c_out is not None else DT_F32, self._stream()),
                    "scaled_add_rmsnorm")

    def qkv_prepare(self, qkv, ctx, cache_layer, group: int, q_out, *, nq: int, nkv: int, d: int, dv: int, dp: int,
                    page_size: int, num_pages: int, store_kv: bool, bias=None, q_norm=None, k_norm=None, eps: float = 0.0,
                    inv_freq=None, rot: int = 0, v_first=None, v_lambda=None, v_out=None, head_norm: bool = False,
                    interleaved: bool = False, q_temp=None):
        """Rows [q | k | v] of the fused projection become attention's inputs: biases, root-mean-square norms over
        the whole q and the whole k part (weights ``q_norm`` / ``k_norm``), rotation of the first ``rot`` dims of
        every head, with ``head_norm`` every q and k head divided by its own root mean square (``eps``) after the rotation,
        v <- (1 - lambda) v + lambda v_first; q to ``q_out`` [T, nq * dp], k and v to the pages as heads of
        dp elements (zeros behind d and dv).  ``v_out``: the values (biases added, unmixed) for later layers.
        ``bias``, ``q_norm`` and ``k_norm`` share one type, float32 or (beside bfloat16 rows) bfloat16.
        With ``head_norm`` AND weights, the weights have ``d`` elements, shared by all heads, and the norm comes before the
        rotation.  ``interleaved``: the rotation pairs dimension 2i with 2i + 1 (else i with i + rot / 2).  ``q_temp`` =
        (coef, every): the query at position p is multiplied by 1 + coef * ln(floor((p + 1) / every) + 1)."""
        if head_norm and (q_norm is not None or k_norm is not None) and (q_norm is None or k_norm is None
                                                                           or q_norm.numel() != d or k_norm.numel() != d):
            raise KernelError("weights beside a norm per head have the head's size, for queries and for keys")
        qt_coef, qt_every = (float(q_temp[0]), int(q_temp[1])) if q_temp else (0.0, 0)
        params = [t for t in (bias, q_norm, k_norm) if t is not None]
        if len({t.dtype for t in params}) > 1:
            raise KernelError("biases and norm weights of the attention rows must share one type")
        pcode = _code(params[0]) if params else DT_F32
        qp, qs = self._rows(qkv, "qkv_prepare")  # (the rows may be the first part of wider ones)
        self._check(self.lib.qkv_prepare(qp, qs, _code(qkv), _p(bias), _p(q_norm), _p(k_norm), pcode, ctypes.c_float(eps),
                                         _p(ctx.positions), _p(ctx.token_entry), _p(ctx.meta), max(group, 0), _p(inv_freq),
                                         int(rot) if inv_freq is not None else 0, _p(v_first), _p(v_lambda), _p(v_out),
                                         _p(q_out), _p(cache_layer), ctx.T, nq, nkv, d, dv, dp, page_size, num_pages,
                                         int(store_kv), int(head_norm), int(interleaved), ctypes.c_float(qt_coef), qt_every,
                                         _p(self.status), self._stream()), "qkv_prepare")

    def narrow(self, x, dtype):
        """Float32 rows in the compute type (rounded once); the same tensor if it has that type already."""
        if x.dtype == dtype:
            return x
        if x.dtype != torch.float32 or dtype != torch.bfloat16:
            raise KernelError(f"narrow: float32 to bfloat16 only, got {x.dtype} to {dtype}")
        out = torch.empty(x.shape, dtype=dtype, device=x.device)
        self._check(self.lib.cast_f32_bf16(_p(x), _p(out), ctypes.c_size_t(x.numel()), self._stream()), "cast_f32_bf16")
        return out

    def polynorm(self, z, coef, eps: float, out, meta):
        """out = a N(z) + b N(z^2) + c N(z^3) + e per row, N(u) = u / sqrt(mean(u^2) + eps); coef = (a, b, c, e)."""
        self._check(self.lib.polynorm(_p(z), _code(z), _p(coef), ctypes.c_float(eps), _p(out), _p(meta), z.shape[0],
                                      z.shape[1], self._stream()), "polynorm")

    def rope_kv_store(self, qkv, positions, token_entry, meta, group: int, inv_freq, cache_layer, num_pages: int,
                      T: int, nq: int, nkv: int, d: int, rot: int, page_size: int, store_kv: bool):
        self._check(self.lib.rope_kv_store(_p(qkv), _code(qkv), _p(positions), _p(token_entry), _p(meta), group,
                                           _p(inv_freq), _p(cache_layer), num_pages, T, nq, nkv, d, rot, page_size,
                                           int(store_kv), _p(self.status), self._stream()), "rope_kv_store")

    def fast_attention(self, dtype, d: int, nq: int, nkv: int, q_stride: int) -> bool:
        """Whether the tensor-core attention kernels take this geometry."""
        return (dtype == torch.bfloat16 and d % 16 == 0 and d <= 256 and nq % nkv == 0 and nq // nkv <= 16
                and q_stride % 8 == 0)

    def attention(self, q, q_stride: int, cache_layer, ctx, group: int, out, nq: int, nkv: int, d: int,
                  page_size: int, num_pages: int, window: int, scale: float, rope=None, chunk: int = 0, sink: bool = False,
                  keep_first: int = 0, softcap: float = 0.0, slopes=None):
        """Attention of the step's queries over what their requests have cached (the step's own
        keys included).  bfloat16 with a head size in steps of 16 up to 256 runs the tensor-core
        kernels (one library per head size, built at first use); anything else, and all of
        float32, runs the plain kernel.  ``rope`` = (inv_freq, rotary_dim, store_kv): only for decode
        steps on the fast path (see ``fast_attention``); the queries are then still unrotated and the
        kernel rotates them, and writes the new key and value, itself.  ``chunk`` > 0: a query sees only the keys of
        its own chunk of that many positions (chunks counted from position 0 of the request).  ``sink``: the softmax
        has one more term in its denominator, a key of score 0 without a value.  ``keep_first`` (beside a window): the
        first so many keys of a request stay visible behind the window.  ``softcap`` > 0: a score s becomes softcap *
        tanh(s / softcap).  ``slopes`` (float32, one per query head): slopes[h] * (query position - key position) is
        taken off the score."""
        T, S = ctx.T, ctx.S
        if slopes is not None and (slopes.dtype != torch.float32 or slopes.numel() != nq or not slopes.is_contiguous()):
            raise KernelError("distance slopes are one contiguous float32 number per query head")
        # a learned sink: one float32 score per query head (a tensor) instead of the score 0 (True)
        sinks = sink if torch.is_tensor(sink) else None
        sink = sinks is not None or bool(sink)
        if sinks is not None and (sinks.dtype != torch.float32 or sinks.numel() != nq or not sinks.is_contiguous()):
            raise KernelError("learned sinks are one contiguous float32 score per query head")
        keep_first = int(keep_first) if window and not chunk else 0
        scored = bool(keep_first or softcap or slopes is not None)
        if scored and rope is not None:
            raise KernelError("the fused rotation does not go with kept first tokens, a score cap or distance slopes")
        extra = (keep_first, ctypes.c_float(float(softcap)), _p(slopes))
        if scored and not self.scored_fast_attention:  # (a test lever: the plain kernel in both number formats)
            self._attention_scores(q, q_stride, cache_layer, ctx, group, out, nq, nkv, d, page_size, num_pages, window, scale,
                                   chunk, sinks if sinks is not None else sink, keep_first, float(softcap), slopes)
            return
        if (chunk or sink) and self.fast_attention(q.dtype, d, nq, nkv, q_stride) and not self.masked_fast_attention:
            self._attention_scores(q, q_stride, cache_layer, ctx, group, out, nq, nkv, d, page_size, num_pages, window, scale,
                                   chunk, sinks if sinks is not None else sink, keep_first, float(softcap), slopes)
            return

        if rope is not None and not (ctx.decode_only and self.fast_attention(q.dtype, d, nq, nkv, q_stride)):
            raise KernelError("fused rotation exists for decode steps on the bfloat16 fast path only")
        if self.fast_attention(q.dtype, d, nq, nkv, q_stride):
            lib = self._attention_library(d)
            if ctx.decode_only:
                inv_freq, rot, store = rope if rope is not None else (None, 0, False)
                # a chunk bounds the keys of a request and a sink is one more partial result: both go with fixed splits
                flat_blocks = 0 if (chunk or sink or scored) else self._decode_flat_blocks(lib, d, S, nkv)
                if flat_blocks:
                    # large batch: as many blocks as the GPU holds share all key tiles evenly
                    n = lib.attn_decode_flat_scratch_floats(S, nq, nkv, flat_blocks)
                    scratch = torch.empty(n, dtype=torch.float32, device=q.device)
                    if S * nkv > self._counters.numel():
                        raise KernelError(f"decode attention: {S} requests x {nkv} heads exceed the split counters")
                    self._check(lib.attn_decode_flat(_p(q), q_stride, _p(cache_layer), _p(ctx.meta), group,
                                                     _p(ctx.cu_tokens), _p(ctx.positions), _p(out), _p(scratch),
                                                     _p(self._counters), _p(inv_freq), rot, int(store), S, nq, nkv,
                                                     page_size, num_pages, window, ctypes.c_float(scale), flat_blocks,
                                                     _p(self.status), self._stream()), "attn_decode_flat")
                    return
                seen = min(ctx.max_context, chunk) if chunk else ctx.max_context  # most keys a request reads
                if window:
                    seen = min(seen, window + keep_first)
                splits = self.decode_splits(S, nkv, seen, lib.attn_decode_blocks_per_sm())
                # the splits merge inside a thread-block cluster when they fit one, else through scratch
                if S <= SKINNY_MAX_ROWS:
                    self._prefetch_next_weight(S)
                cluster = self.decode_cluster and 1 < splits <= lib.attn_decode_max_cluster()
                n = 0 if cluster else lib.attn_decode_scratch_floats(S, nq, splits)
                scratch = torch.empty(n, dtype=torch.float32, device=q.device) if n else None
                if not cluster and S * nkv > self._counters.numel():
                    raise KernelError(f"decode attention: {S} requests x {nkv} heads exceed the split counters")
                self._check(lib.attn_decode_scores(_p(q), q_stride, _p(cache_layer), _p(ctx.meta), group, _p(ctx.cu_tokens),
                                                   _p(ctx.positions), _p(out), _p(scratch), _p(self._counters), _p(inv_freq),
                                                   rot, int(store), S, nq, nkv, page_size, num_pages,
                                                   window, int(chunk), int(bool(sink)), _p(sinks), ctypes.c_float(scale), splits,
                                                   int(cluster), ctx.max_context, *extra, _p(self.status), self._stream()),
                            "attn_decode")
            elif not keep_first and self._prefill_tc(d, page_size, nq, nkv) is not None:
                # (a window that keeps first keys is the mma.sync kernel's: its kept keys are tiles of their own)
                tc = self._prefill_tc(d, page_size, nq, nkv)
                self._check(tc.attn_prefill_tc_scores(_p(q), q_stride, _p(cache_layer), _p(ctx.meta), group, _p(ctx.cu_tokens),
                                                      _p(ctx.context_lens), _p(out), S, ctx.max_tokens_per_entry, nq, nkv,
                                                      page_size, num_pages, window, int(chunk), int(bool(sink)), _p(sinks),
                                                      ctypes.c_float(scale), ctx.max_context, ctypes.c_float(float(softcap)),
                                                      _p(slopes), _p(self.status), self._stream()),
                            "attn_prefill_tc")
            else:
                self._check(lib.attn_prefill_scores(_p(q), q_stride, _p(cache_layer), _p(ctx.meta), group, _p(ctx.cu_tokens),
                                                    _p(ctx.context_lens), _p(out), S, ctx.max_tokens_per_entry, nq, nkv,
                                                    page_size, num_pages, window, int(chunk), int(bool(sink)), _p(sinks),
                                                    ctypes.c_float(scale), ctx.max_context, *extra, _p(self.status), self._stream()),
                            "attn_prefill")
            return
        self._attention_scores(q, q_stride, cache_layer, ctx, group, out, nq, nkv, d, page_size, num_pages, window, scale, chunk,
                               sinks if sinks is not None else sink, keep_first, float(softcap), slopes)

    def _attention_scores(self, q, q_stride, cache_layer, ctx, group, out, nq, nkv, d, page_size, num_pages, window, scale,
                          chunk, sink, keep_first, softcap, slopes) -> bool:
        """The plain attention kernel (both number formats, any head size up to 512), with every option."""
        sinks = sink if torch.is_tensor(sink) else None
        if d > 512:
            raise KernelError(f"head size {d} is not supported (at most 512)")
        self._check(self.lib.attn_generic_scores(_p(q), q_stride, _p(cache_layer), _code(q), _p(ctx.meta), group,
                                                 _p(ctx.token_entry), _p(ctx.positions), _p(out), ctx.T, nq, nkv, d, page_size,
                                                 num_pages, window, int(chunk), int(sinks is not None or bool(sink)), _p(sinks),
                                                 ctypes.c_float(scale), keep_first, ctypes.c_float(softcap), _p(slopes),
                                                 _p(self.status), self._stream()), "attn_generic")
        return True

    # ------------------------------------------------------------------ blocks that norm a sublayer's result and gate it
    def norm_shift(self, resid, w, eps: float, ctx, *, shift=None, state=None, h=None, hs=None, last=None):
        """h[t] = rmsnorm(resid[t]) * w and hs[t] = h[t] + (h[t - 1] - h[t]) * shift, h[t - 1] being the normed row of the
        token before in the same request: of this step, or the row kept in ``state`` (float32 [slots, H] with a slot
        stride), or zeros at position 0.  ``last`` (float32 [S, H]) receives every entry's last normed row, which
        ``gated_norm_add`` moves into the state once nothing reads the old one any more.  Without ``shift`` hs = h."""
        H = resid.shape[1]
        outs = [t for t in (h, hs) if t is not None]
        if not outs or len({t.dtype for t in outs}) > 1:
            raise KernelError("norm_shift writes h, hs or both, of one type")
        stride = ctypes.c_longlong(state.stride(0)) if state is not None else ctypes.c_longlong(0)
        if state is not None and (state.dtype != torch.float32 or state.dim() != 2 or state.stride(1) != 1 or state.shape[1] != H):
            raise KernelError("the kept row is float32 [slots, H] with contiguous rows")
        self._check(self._mixers().norm_shift(_p(resid), _p(w), ctypes.c_float(eps), _p(shift), _p(state), stride, _p(h), _p(hs),
                                              _code(outs[0]), _p(last), _p(ctx.meta), _p(ctx.positions), _p(ctx.token_entry),
                                              _p(ctx.cu_tokens), _p(ctx.state_slots), ctx.T, H, self._stream()), "norm_shift")

    def gated_norm_add(self, resid, pending, gate, gate_bias, w, eps: float, ctx, *, next_norm=None, keep=None):
        """resid[t] += rmsnorm(y[t] * sigmoid(gate[t] + gate_bias)) * w with y = mult * (f0 t0 + f1 t1 + ...) + vector, the
        terms, weights, factor and vector of ``pending`` (a ``PendingSum``; up to four terms of one type).  ``gate``: the
        gate's logits [T, H] (float32, or the terms' type), ``gate_bias`` float32 [H] or None.  ``next_norm`` = (w2, eps2,
        out): also out[t] = rmsnorm(resid[t]) * w2, the next sublayer's input.  ``keep`` = (last, state): every entry's row
        of ``last`` moves into its slot of ``state`` (see ``norm_shift``)."""
        H = resid.shape[1]
        terms = list(pending.terms)
        if not 0 < len(terms) <= 4 or len({t.dtype for t in terms}) > 1:
            raise KernelError("a gated sum has one to four terms, of one type")
        if pending.rows is not None:
            raise KernelError("a gated sum has terms, weights, a factor and a vector only")
        ptrs = (ctypes.c_void_p * 4)(*[t.data_ptr() for t in terms])
        facs = (ctypes.c_float * 4)(*pending.weights())
        w2, eps2, out = next_norm if next_norm is not None else (None, 0.0, None)
        last, state = keep if keep is not None else (None, None)
        stride = ctypes.c_longlong(state.stride(0)) if state is not None else ctypes.c_longlong(0)
        self._check(self._mixers().gated_norm_add(_p(resid), len(terms), ptrs, facs, _code(terms[0]), ctypes.c_float(pending.mult),
                                                  _p(pending.vector), _p(gate), _code(gate), _p(gate_bias), _p(w), ctypes.c_float(eps),
                                                  _p(w2), ctypes.c_float(eps2), _p(out), _code(out) if out is not None else _code(terms[0]),
                                                  _p(last), _p(state), stride, _p(ctx.meta), _p(ctx.token_entry), _p(ctx.cu_tokens),
                                                  _p(ctx.state_slots), ctx.T, H, self._stream()), "gated_norm_add")

    def clamped_glu(self, gu, out, limit: float, alpha: float, meta):
        """out = g * sigmoid(alpha * g) * (u + 1) with g = min(gate, limit), u = clamp(up, -limit, limit); ``gu`` [T, 2F], the
        gate's columns first."""
        self._check(self._mixers().clamped_glu(_p(gu), _p(out), _code(gu), _p(meta), gu.shape[0], out.shape[1], ctypes.c_float(limit),
                                               ctypes.c_float(alpha), self._stream()), "clamped_glu")

    def head_gate(self, y, gate, meta):
        """y[t, h, :] *= sigmoid(gate[t, h]) in place: ``y`` [T, heads, n] with a contiguous last axis, ``gate`` [T, heads] a
        slice of wider rows."""
        T, heads, n = y.shape
        yp, yt, yh = self._heads(y, "head_gate")
        gp, gs = self._rows(gate, "head_gate")
        self._check(self._mixers().head_gate(yp, yt, yh, gp, gs, _code(y), _p(meta), T, heads, n, self._stream()), "head_gate")

    def row_norm_gate(self, o, gate, w, eps: float, out, meta, kind: str = "sigmoid"):
        """out[t] = o[t] / sqrt(mean(o[t]^2) + eps) * w * gate_fn(gate[t]): ``o`` float32 [T, n], ``gate`` a slice of wider rows,
        ``w`` float32 [n]; ``kind``: "sigmoid" or "silu"."""
        gp, gs = self._rows(gate, "row_norm_gate")
        self._check(self._mixers().row_norm_gate(_p(o), gp, _code(gate), gs, _p(w), ctypes.c_float(eps), _p(out), _p(meta), o.shape[0],
                                                 o.shape[1], {"sigmoid": 0, "silu": 1}[kind], self._stream()), "row_norm_gate")

    def scale_softcap(self, logits, scale: float, cap: float, meta):
        """logits <- cap * tanh(logits * scale / cap) in place (cap 0: logits * scale); float32 [rows, n]."""
        self._check(self._mixers().scale_softcap(_p(logits), _p(meta), logits.shape[0], logits.shape[1], ctypes.c_float(scale),
                                                 ctypes.c_float(cap), self._stream()), "scale_softcap")

    # ------------------------------------------------------------------ parallel blocks, state-space mixers, latent attention, experts
    def _mixers(self):
        lib = getattr(self, "_mixer_lib", None)
        if lib is None:
            lib = self._mixer_lib = build.load_library("mixers", MIXER_SOURCES, cuda=True)
            lib.ssm_scan_scratch_floats.restype = ctypes.c_size_t
            lib.kernels_set_pdl(int(self.pdl))
        return lib

    @staticmethod
    def _rows(t, what: str):
        """(pointer, elements from row to row) of a 2-d slice whose rows are contiguous."""
        if t.dim() != 2 or t.stride(1) != 1:
            raise KernelError(f"{what}: rows must be contiguous, got strides {t.stride()}")
        return _p(t), ctypes.c_longlong(t.stride(0))

    @staticmethod
    def _heads(t, what: str):
        """(pointer, token stride, head stride) of a [T, heads, n] slice whose last axis is contiguous."""
        if t.dim() != 3 or t.stride(2) != 1:
            raise KernelError(f"{what}: the last axis must be contiguous, got strides {t.stride()}")
        return _p(t), ctypes.c_longlong(t.stride(0)), ctypes.c_longlong(t.stride(1))

    def sum_rmsnorm(self, resid, pending, w, eps: float, out, meta, n: int, rows=None, second=None):
        """resid += mult * (f0 t0 + f1 t1 + ...) + pending.rows + pending.vector, each optional, in float32 (up to four
        terms, their weights ``pending.factors``, 1 if none); out = rmsnorm(resid) * w if ``out`` is given; ``second`` =
        (w2, eps2, out2): the same rows normed once more with another weight.  With ``rows`` the sum and the norm are
        taken at those rows only and resid is left as it is."""
        terms = list(pending.terms) if pending is not None else []
        if len(terms) > 4 or len({t.dtype for t in terms}) > 1:
            raise KernelError("a pending sum has at most four terms, of one type")
        factors = list(pending.weights()) if pending is not None else []
        tcode = _code(terms[0]) if terms else DT_F32
        w2, eps2, out2 = second if second is not None else (None, 0.0, None)
        ptrs = (ctypes.c_void_p * 4)(*[t.data_ptr() for t in terms])
        facs = (ctypes.c_float * 4)(*factors)
        self._check(self._mixers().sum_rmsnorm_terms(_p(resid), len(terms), ptrs, facs, tcode,
                                                     ctypes.c_float(pending.mult if pending else 1.0),
                                                     _p(pending.rows if pending else None), _p(pending.vector if pending else None),
                                                     _p(rows), _p(w), ctypes.c_float(eps), _p(out), _p(w2), ctypes.c_float(eps2),
                                                     _p(out2), _code(out) if out is not None else DT_F32, _p(meta), n,
                                                     resid.shape[-1], self._stream()), "sum_rmsnorm")

    def activation(self, z, out, kind: str, meta):
        """out = act(z) element by element; ``kind``: "gelu_tanh", or "relu2" (the square of relu)."""
        code = {"gelu_tanh": 0, "relu2": 1}[kind]
        self._check(self._mixers().activation_rows(_p(z), _p(out), _code(z), _p(meta), z.shape[0], z.shape[1], code,
                                                   self._stream()), "activation_rows")

    def causal_conv_act(self, u, w, bias, state, ctx, out, *, act: str = "silu") -> bool:
        """out[t] = act(bias + sum_j w[j] * u[t - taps + 1 + j]) over the rows of each request, zeros before its start; ``u``
        a slice of wider rows, ``w`` float32 [taps, C], ``bias`` float32 [C] or None; rows before the step's portion come
        from ``state`` (float32 [slots, taps - 1, C], the row of position p at place p mod (taps - 1)).  Returns whether
        the state has been updated too (decode steps, where the thread that read a channel's ring also owns the new
        row's place); if not, ``causal_conv_save`` writes it afterwards."""
        taps, C = w.shape
        up, us = self._rows(u, "causal_conv_act")
        lib = self._mixers()
        saves = bool(taps > 1 and ctx.decode_only and ctx.T == ctx.S and
                     lib.causal_conv_act_saves(up, _code(u), us, _p(w), _p(bias), _p(state), self._slot_stride(state), _p(out), C))
        self._check(lib.causal_conv_act(up, _code(u), us, _p(w), _p(bias), _p(state), self._slot_stride(state), _p(out),
                                        _p(ctx.meta), _p(ctx.positions), _p(ctx.token_entry), _p(ctx.cu_tokens),
                                        _p(ctx.state_slots), ctx.T, C, taps, {"none": 0, "silu": 1}[act], int(saves),
                                        self._stream()), "causal_conv_act")
        return saves or taps == 1

    def causal_conv_save(self, u, state, ctx, taps: int):
        """The last taps - 1 rows of u of every entry go to its state (see ``causal_conv_act``)."""
        if taps > 1:
            up, us = self._rows(u, "causal_conv_save")
            self._check(self._mixers().causal_conv_save(up, _code(u), us, _p(state), self._slot_stride(state), _p(ctx.meta),
                                                        _p(ctx.positions), _p(ctx.token_entry), _p(ctx.cu_tokens),
                                                        _p(ctx.state_slots), ctx.T, u.shape[1], taps, self._stream()),
                        "causal_conv_save")

    SCAN_CHUNK = 64        # tokens of a chunk when a long portion's recurrence is cut into chunks that run side by side
    SCAN_CHUNK_FROM = 128  # ... which happens from this many tokens of the step's longest entry on

    def ssm_scan(self, xbc, dt, dt_bias, a_log, d_skip, state, ctx, y, *, heads: int, head_dim: int, nstate: int, groups: int):
        """The state-space recurrence of every entry's tokens: rows of ``xbc`` are [x | B | C], ``dt`` a slice of wider
        rows (softplus(dt + dt_bias) is taken here), ``state`` float32 [slots, heads, nstate, head_dim] (read and
        updated), ``y`` float32 [T, heads * head_dim]."""
        if state.dim() != 4 or state[0].is_contiguous() is False or state.dtype != torch.float32:
            raise KernelError("a recurrence state is float32 [slots, heads, rows, columns] with contiguous slots")
        dp, ds = self._rows(dt, "ssm_scan")
        lib = self._mixers()
        longest = ctx.max_tokens_per_entry
        chunk = self.SCAN_CHUNK if longest >= self.SCAN_CHUNK_FROM else 0
        while chunk and longest // chunk > 256:
            chunk *= 2
        chunks = -(-longest // chunk) if chunk else 1
        scratch = (torch.empty(lib.ssm_scan_scratch_floats(ctx.S, heads, head_dim, nstate, chunks), dtype=torch.float32,
                               device=y.device) if chunk else None)
        self._check(lib.ssm_scan(_p(xbc), _code(xbc), xbc.stride(0), dp, ds, _p(dt_bias), _p(a_log), _p(d_skip), _p(state),
                                 ctypes.c_longlong(state.stride(0)), _p(y), _p(ctx.meta), _p(ctx.cu_tokens), _p(ctx.state_slots),
                                 ctx.S, heads, head_dim, nstate, groups, chunk, chunks, _p(scratch), self._stream()), "ssm_scan")
        if chunk:
            self.launches += 2

    def gated_group_norm(self, y, z, w, groups: int, eps: float, out, meta):
        """out = v / sqrt(mean(v^2) + eps) * w with v = y * silu(z), the mean over each of ``groups`` equal parts of a row;
        ``y`` float32 [T, n], ``z`` a slice of wider rows."""
        zp, zs = self._rows(z, "gated_group_norm")
        self._check(self._mixers().gated_group_norm(_p(y), zp, _code(z), zs, _p(w), ctypes.c_float(eps), _p(out), _p(meta),
                                                    y.shape[0], y.shape[1], groups, self._stream()), "gated_group_norm")

    def rms_rows(self, x, w, eps: float, out, meta):
        """out = x * rsqrt(mean(x^2) + eps) * w row by row; ``x`` a slice of wider rows, ``w`` float32."""
        xp, xs = self._rows(x, "rms_rows")
        self._check(self._mixers().rms_rows(xp, _code(x), xs, _p(w), ctypes.c_float(eps), _p(out), _p(meta), x.shape[0], x.shape[1],
                                            self._stream()), "rms_rows")

    HEAD_LINEAR_LIBRARY_ROWS = 64  # from this many rows on, a bfloat16 map per head is a batched library product

    def head_linear(self, x, w, out, meta, gate=None):
        """out[t, h] = w[h] x[t, h] (times sigmoid(gate[t, h]) if given): x [T, heads, K], out and gate [T, heads, N] slices
        with a contiguous last axis, w [heads, N, K] contiguous."""
        heads, N, K = w.shape
        T = x.shape[0]
        lib = self._mixers()
        op, ot, oh = self._heads(out, "head_linear")
        gp, gt, gh = self._heads(gate, "head_linear") if gate is not None else (None, ctypes.c_longlong(0), ctypes.c_longlong(0))
        if x.dtype == torch.bfloat16 and T >= self.HEAD_LINEAR_LIBRARY_ROWS:
            out.copy_(torch.bmm(x.transpose(0, 1), w.transpose(1, 2)).transpose(0, 1))
            if gate is not None:
                self._check(lib.sigmoid_gate(op, ot, oh, gp, gt, gh, _code(out), _p(meta), T, heads, N, self._stream()),
                            "sigmoid_gate")
            return
        xp, xt, xh = self._heads(x, "head_linear")
        self._check(lib.head_linear(xp, xt, xh, _p(w), op, ot, oh, gp, gt, gh, _code(x), _p(meta), T, heads, K, N,
                                    self._stream()), "head_linear")

    def latent_rows(self, q_rot, q_abs, dkv, norm_w, eps: float, ctx, cache_layer, group: int, q_out, *, heads: int,
                    kv_rank: int, rot_dim: int, padded: int, page_size: int, num_pages: int, store: bool, inv_freq=None,
                    rotary_dims: int = 0):
        """The rows of latent attention.  The cached vector [rmsnorm(dkv[:kv_rank]) * norm_w | rotated dkv[kv_rank:] |
        zeros] of ``padded`` elements goes to the key plane and the value plane of the token's page; the queries become
        [q_abs[h] | rotated q_rot[h] | zeros] in ``q_out`` [T, heads * padded].  Rotation: of the first ``rotary_dims``
        dimensions, 2i pairs with 2i + 1, angle position * inv_freq[i]."""
        qp, qt, qh = self._heads(q_rot, "latent_rows")
        dp, ds = self._rows(dkv, "latent_rows")
        if not q_abs.is_contiguous():
            raise KernelError("latent_rows: q_abs must be contiguous")
        self._check(self._mixers().latent_rows(qp, qt, qh, _p(q_abs), dp, ds, _p(norm_w), ctypes.c_float(eps), _p(ctx.positions),
                                               _p(ctx.token_entry), _p(ctx.meta), max(group, 0), _p(inv_freq),
                                               int(rotary_dims) if inv_freq is not None else 0, _p(q_out), _p(cache_layer),
                                               _code(q_out), ctx.T, heads, kv_rank, rot_dim, padded, page_size, num_pages,
                                               int(store), _p(self.status), self._stream()), "latent_rows")

    def sigmoid_gate(self, y, gate, meta):
        """y[t, h] *= sigmoid(gate[t, h]) in place: y and gate [T, heads, N] slices with a contiguous last axis."""
        T, heads, N = y.shape
        yp, yt, yh = self._heads(y, "sigmoid_gate")
        gp, gt, gh = self._heads(gate, "sigmoid_gate")
        self._check(self._mixers().sigmoid_gate(yp, yt, yh, gp, gt, gh, _code(y), _p(meta), T, heads, N, self._stream()),
                    "sigmoid_gate")

    # ------------------------------------------------------------------ recurrences with a decay per row
    def _recurrent(self):
        lib = getattr(self, "_recurrent_lib", None)
        if lib is None:
            lib = self._recurrent_lib = build.load_library("recurrent", RECURRENT_SOURCES, cuda=True)
            lib.gla_scan_scratch_floats.restype = ctypes.c_size_t
            lib.selective_scan_scratch_floats.restype = ctypes.c_size_t
            lib.kernels_set_pdl(int(self.pdl))
        return lib

    def _scan_chunks(self, ctx):
        """(tokens of a chunk, chunks of the longest entry) when a long portion's recurrence is cut into chunks of time
        that run side by side; (0, 1): every entry's tokens in order."""
        longest = ctx.max_tokens_per_entry
        chunk = self.SCAN_CHUNK if longest >= self.SCAN_CHUNK_FROM else 0
        while chunk and longest // chunk > 256:
            chunk *= 2
        return chunk, (-(-longest // chunk) if chunk else 1)

    @staticmethod
    def _slot_state(state, shape, what: str):
        if state.dtype != torch.float32 or tuple(state.shape[1:]) != tuple(shape) or not state[0].is_contiguous():
            raise KernelError(f"{what}: the state is float32 [slots, {', '.join(map(str, shape))}] with contiguous slots")
        return ctypes.c_longlong(state.stride(0))

    def gla_scan(self, q, k, v, z, z_bias, tau: float, q_scale: float, state, ctx, o, *, heads: int, dim: int, vdim: int,
                 head_decay=None, silu: bool = False):
        """Gated linear attention of every entry's tokens: per head S_t = diag(a_t) S_(t-1) + k_t v_t^T, o_t = S_t^T (q_scale
        q_t), a_t = sigmoid(z_t + z_bias)^(1 / tau).  q, k [T, heads * dim] and v [T, heads * vdim] are slices of wider rows,
        ``z`` float32 [T, heads * dim], ``state`` float32 [slots, heads, dim, vdim] (read and updated), ``o`` float32
        [T, heads * vdim].  ``head_decay`` (float32 [heads]) instead of ``z``: every row of head h decays by the constant
        head_decay[h].  ``silu``: q, k and v pass through SiLU first."""
        lib = self._recurrent()
        slot_stride = self._slot_state(state, (heads, dim, vdim), "gla_scan")
        if o.dtype != torch.float32 or not o.is_contiguous():
            raise KernelError("gla_scan: outputs are float32")
        (qp, qs), (kp, ks), (vp, vs) = (self._rows(t, "gla_scan") for t in (q, k, v))
        if head_decay is not None:
            if z is not None or head_decay.dtype != torch.float32 or head_decay.numel() != heads:
                raise KernelError("gla_scan: a constant decay is one float32 number per head, given instead of logits")
            zp, zs, z_bias, tau = None, ctypes.c_longlong(0), head_decay, 1.0
        else:
            if z.dtype != torch.float32:
                raise KernelError("gla_scan: decay logits are float32")
            zp, zs = self._rows(z, "gla_scan")
        mode = (1 if head_decay is not None else 0) | (2 if silu else 0)
        chunk, chunks = self._scan_chunks(ctx)
        scratch = (torch.empty(lib.gla_scan_scratch_floats(ctx.S, heads, dim, vdim, chunks), dtype=torch.float32, device=o.device)
                   if chunk else None)
        self._check(lib.gla_scan_mode(qp, qs, kp, ks, vp, vs, _code(q), zp, zs, _p(z_bias), ctypes.c_float(tau), ctypes.c_float(q_scale),
                                      _p(state), slot_stride, _p(o), _p(ctx.meta), _p(ctx.cu_tokens), _p(ctx.state_slots), ctx.S,
                                      heads, dim, vdim, chunk, chunks, _p(scratch), mode, self._stream()), "gla_scan")
        if chunk:
            self.launches += 2

    def head_norm_gate(self, o, gate, w, eps: float, out, meta, heads: int):
        """out[t, h] = o[t, h] / sqrt(mean(o[t, h]^2) + eps) * w * silu(gate[t, h]): ``o`` float32 [T, heads * P], ``gate`` a
        slice of wider rows, ``w`` float32 [P] (the same for every head)."""
        gp, gs = self._rows(gate, "head_norm_gate")
        self._check(self._recurrent().head_norm_gate(_p(o), gp, _code(gate), gs, _p(w), ctypes.c_float(eps), _p(out), _p(meta),
                                                     o.shape[0], heads, o.shape[1] // heads, self._stream()), "head_norm_gate")

    def selective_scan(self, u, dt_raw, dt_bias, bc, zg, a_log, d_skip, state, ctx, out, *, inner: int, nstate: int):
        """The selective scan of every entry's tokens: per channel c and state n, S[c, n] <- exp(dt_c A[c, n]) S[c, n] +
        dt_c u_c B_n with dt = softplus(dt_raw + dt_bias) and A = -exp(a_log); out = (S C + d_skip u) * silu(zg).  ``u`` and
        ``zg`` [T, inner] and ``bc`` [T, 2 * nstate] (B, then C) are slices of wider rows, ``dt_raw`` float32 [T, inner],
        ``state`` float32 [slots, inner, nstate] (read and updated), ``out`` [T, inner] in the type of ``u``."""
        lib = self._recurrent()
        slot_stride = self._slot_state(state, (inner, nstate), "selective_scan")
        if dt_raw.dtype != torch.float32 or not dt_raw.is_contiguous() or not out.is_contiguous() or out.dtype != u.dtype:
            raise KernelError("selective_scan: step sizes are contiguous float32, the output has the inputs' type")
        (up, us), (bp, bs), (zp, zs) = (self._rows(t, "selective_scan") for t in (u, bc, zg))
        chunk, chunks = self._scan_chunks(ctx)
        scratch = (torch.empty(lib.selective_scan_scratch_floats(ctx.S, inner, nstate, chunks), dtype=torch.float32, device=out.device)
                   if chunk else None)
        self._check(lib.selective_scan(up, us, _p(dt_raw), _p(dt_bias), bp, bs, zp, zs, _code(u), _p(a_log), _p(d_skip), _p(state),
                                       slot_stride, _p(out), _p(ctx.meta), _p(ctx.cu_tokens), _p(ctx.state_slots), ctx.S, inner,
                                       nstate, chunk, chunks, _p(scratch), self._stream()), "selective_scan")
        if chunk:
            self.launches += 2

    def moe_route(self, h, w_router, ids, wts, meta, bias=None, over_chosen: bool = False):
        """Per token: float32 logits w_router h (+ ``bias``, float32 [experts]), softmax over all experts, the ids.shape[1]
        largest scores (ties to the lower index) into ``ids`` (int32) and those scores divided by their sum (+ 1e-20) into
        ``wts`` (float32).  ``over_chosen``: the weights are the softmax over the chosen experts' logits alone."""
        E, H = w_router.shape
        self._check(self._mixers().moe_route_biased(_p(h), _code(h), _p(w_router), _p(bias), int(over_chosen), _p(ids), _p(wts),
                                                    _p(meta), h.shape[0], H, E, ids.shape[1], self._stream()), "moe_route")

    MOE_PAIR_ROWS = 64       # up to this many (token, choice) pairs, bfloat16: a pair at a time
    MOE_LIBRARY_ROWS = 256   # from this many pairs on, bfloat16: the library's grouped products
    moe_library = hasattr(torch, "_grouped_mm")  # (a test lever too)

    def moe_experts(self, h, ids, wts, w_gate_up, w_down, shared, out, meta):
        """out[t] = sum_k wts[t, k] * expert ids[t, k] of h[t] (+ shared[t]); an expert is down(silu(gate x) * up x) with
        ``w_gate_up`` [E, 2F, H] (gate rows first) and ``w_down`` [E, H, F].  The (token, choice) pairs are sorted by expert
        on the device and the two linears run as grouped products over that order: on the engine's own tile kernel
        (float32 always: every output's order of summation is then the same for any batch), or, in bfloat16, a pair at a
        time for a handful of pairs and through the library's grouped product for many."""
        T, top = ids.shape
        E, F2, H = w_gate_up.shape
        F = F2 // 2
        lib, dev = self._mixers(), h.device
        pairs, bf = T * top, h.dtype == torch.bfloat16
        act = torch.empty((pairs, F), dtype=h.dtype, device=dev)
        if bf and pairs <= self.MOE_PAIR_ROWS and H % 8 == 0 and F % 8 == 0 and max(H, F) * 2 <= 96 * 1024:
            # a handful of pairs (decode steps): every pair streams its expert's rows itself, no sorting
            y = torch.empty((pairs, H), dtype=torch.float32, device=dev)
            self._check(lib.moe_pair_ff(_p(h), _p(w_gate_up), _p(act), _p(w_down), _p(y), _p(ids), _p(meta), T, top, H, F,
                                        self._stream()), "moe_pair_ff")
            self.launches += 1
            self._check(lib.moe_combine(_p(y), DT_F32, None, _p(wts), _p(shared), _p(out), _code(out), _p(meta), T, top, H,
                                        self._stream()), "moe_combine")
            return
        offsets = torch.empty(E + 1, dtype=torch.int32, device=dev)
        order = torch.empty(pairs, dtype=torch.int32, device=dev)
        place = torch.empty(pairs, dtype=torch.int32, device=dev)
        self._check(lib.moe_sort(_p(ids), _p(offsets), _p(order), _p(place), _p(meta), top, E, self._stream()), "moe_sort")
        if bf and pairs >= self.MOE_LIBRARY_ROWS and self.moe_library and H % 8 == 0 and F % 8 == 0:
            # many pairs: rows gathered in sorted order, the two products as the library's grouped products over the
            # experts' stretches (offsets on the device: no host round trip), like the many-row linears
            xs = torch.empty((pairs, H), dtype=h.dtype, device=dev)
            self._check(lib.moe_gather_rows(_p(h), _p(xs), _p(order), _p(meta), T, top, H * 2, self._stream()), "moe_gather_rows")
            ends = offsets[1:]
            try:
                gu = torch._grouped_mm(xs, w_gate_up.transpose(1, 2), offs=ends)
                self.silu_mul(gu, act, None, pairs, F)
                y = torch._grouped_mm(act, w_down.transpose(1, 2), offs=ends)
            except (RuntimeError, TypeError, NotImplementedError):
                y = None  # the library refuses these sizes or strides: the engine's own grouped kernel from now on
                self.moe_library = False
            if y is not None:
                self._check(lib.moe_combine(_p(y), DT_BF16, _p(place), _p(wts), _p(shared), _p(out), _code(out), _p(meta), T, top,
                                            H, self._stream()), "moe_combine")
                return
        y = torch.empty((pairs, H), dtype=torch.float32, device=dev)
        self._check(lib.moe_grouped_ff(_p(h), _p(w_gate_up), _p(act), _p(w_down), _p(y), _p(offsets), _p(order), _code(h), T, top,
                                       E, H, F, self._stream()), "moe_grouped_ff")
        self.launches += 1
        self._check(lib.moe_combine(_p(y), DT_F32, None, _p(wts), _p(shared), _p(out), _code(out), _p(meta), T, top, H,
                                    self._stream()), "moe_combine")

    # ------------------------------------------------------------------ whole layers of a decode step
    def _decode_stack_library(self, d: int):
        lib = self._stack_libs.get(d)
        if lib is None:
            lib = build.load_library(f"decode_stack_d{d}", DECODE_STACK_SOURCES, cuda=True, defines={"HEAD_DIM": d})
            lib.decode_stack_scratch_floats.restype = ctypes.c_size_t
            if lib.decode_stack_head_dim() != d:
                raise KernelError(f"decode stack library was built for head size {lib.decode_stack_head_dim()}, wanted {d}")
            self._stack_libs[d] = lib
        return lib

    def decode_stack_layers(self, layers, *, d: int, hidden: int, intermediate: int, nq: int, nkv: int, page_size: int,
                            num_pages: int) -> torch.Tensor:
        """The layer kernel's descriptors on the device, one per dict of ``layers`` (tensors ``w_qkv``, ``w_o``,
        ``w_gate_up``, ``w_down``, ``norm1``, ``norm2``, ``inv_freq``, ``cache``; bool ``store_kv``)."""
        lib = self._decode_stack_library(d)
        size = int(lib.decode_stack_layer_bytes())
        host = torch.zeros(len(layers) * size, dtype=torch.uint8)
        for i, ly in enumerate(layers):
            err = lib.decode_stack_fill_layer(ctypes.c_void_p(host.data_ptr() + i * size), _p(ly["w_qkv"]), _p(ly["w_o"]),
                                              _p(ly["w_gate_up"]), _p(ly["w_down"]), _p(ly["norm1"]), _p(ly["norm2"]),
                                              _p(ly["inv_freq"]), _p(ly["cache"]), int(ly["store_kv"]), hidden, intermediate,
                                              nq, nkv, page_size, num_pages)
            if err:
                raise KernelError(f"decode_stack_fill_layer: error {err} (widths must be multiples of 64)")
        return host.to(self.device)

    def decode_stack_record_clocks(self, d: int, buffer: Optional[torch.Tensor]) -> None:
        """For measurements: the next launches of the layer kernel leave the global clock after every phase and every
        barrier of every layer in ``buffer`` (int64 [blocks, layers, 10]; None: off).  Reading that clock costs each
        block a few hundred nanoseconds a time."""
        self._decode_stack_library(d).decode_stack_set_times(_p(buffer))

    def decode_stack_blocks(self, d: int, rows: int, hidden: int) -> int:
        """Blocks the layer kernel would run with for ``rows`` rows of width ``hidden`` (the larger of the model's
        width and heads x head size; 0: it does not take them)."""
        key = (d, rows <= 8, hidden)
        n = self._stack_blocks.get(key)
        if n is None:
            ok = d % 16 == 0 and 16 <= d <= 256 and hidden % 8 == 0
            n = self._stack_blocks[key] = int(self._decode_stack_library(d).decode_stack_blocks(rows, hidden)) if ok else 0
        return n if rows <= SKINNY_MAX_ROWS else 0

    def decode_stack(self, layers, num_layers: int, resid, delta, arrivals, ctx, group: int, *, hidden: int, intermediate: int,
                     nq: int, nkv: int, d: int, rot: int, window: int, page_size: int, num_pages: int, eps: float,
                     scale: float, all_store_kv: bool = True):
        """``num_layers`` pre-norm layers (RMSNorm, rotary attention over the paged cache, SwiGLU) of a decode step in
        one launch (kernels/decode_stack.cu): resid [rows, hidden] float32 is updated in place, ``delta`` added first."""
        lib = self._decode_stack_library(d)
        M = ctx.T
        blocks = self.decode_stack_blocks(d, M, max(hidden, nq * d))
        if not blocks or ctx.S != M or not ctx.decode_only:
            raise KernelError("the decode layer kernel takes decode steps of at most 16 rows")
        if M * nkv > self._counters.numel():
            raise KernelError(f"decode layers: {M} requests x {nkv} heads exceed the split counters")
        dev = resid.device
        qkv = torch.empty((M, (nq + 2 * nkv) * d), dtype=torch.bfloat16, device=dev)
        out = torch.empty((M, nq * d), dtype=torch.bfloat16, device=dev)
        act = torch.empty((M, intermediate), dtype=torch.bfloat16, device=dev)
        xw = torch.empty((M, hidden), dtype=torch.bfloat16, device=dev)
        ss_part = torch.empty(-(-hidden // 16) * 16, dtype=torch.float32, device=dev)
        scratch = torch.empty(lib.decode_stack_scratch_floats(M, nq, nkv, blocks), dtype=torch.float32, device=dev)
        self._check(lib.decode_stack(_p(layers), num_layers, _p(resid), _p(delta), _p(qkv), _p(out), _p(act), _p(xw), _p(ss_part), _p(scratch),
                                     _p(self._counters), _p(arrivals), _p(ctx.meta), group, _p(ctx.cu_tokens), _p(ctx.positions),
                                     M, ctx.S, hidden, intermediate, nq, nkv, rot, window, page_size, num_pages,
                                     ctypes.c_float(eps), ctypes.c_float(scale), int(all_store_kv), _p(self.status), self._stream()),
                    "decode_stack")

    def _decode_flat_blocks(self, lib, d: int, S: int, nkv: int) -> int:
        """Grid size of the flat decode kernel if this batch should take it (at least half as many (request,
        head group) pairs as blocks the GPU holds: below that, fixed splits in clusters fill the GPU as well
        and merge faster), else 0."""
        if not self.decode_flat:
            return 0
        if self.decode_flat_forced:
            return self.decode_flat_forced
        key = (d, S)
        blocks = self._flat_blocks.get(key)
        if blocks is None:
            blocks = self._flat_blocks[key] = int(lib.attn_decode_flat_blocks(S))
        return blocks if blocks and 2 * S * nkv >= blocks else 0

    def _prefill_tc(self, d: int, page_size: int, nq: int, nkv: int):
        """The tcgen05 prefill attention library for this geometry, or None (then the mma.sync kernel runs)."""
        if d not in ATTENTION_TC_HEAD_DIMS or not self.tc_attention:
            return None
        lib = self._attn_tc_libs.get(d)
        if lib is None:
            lib = build.load_library(f"attention_tc_d{d}", ATTENTION_TC_SOURCES, cuda=True, defines={"HEAD_DIM": d})
            if lib.attn_tc_head_dim() != d:
                raise KernelError(f"tcgen05 attention library was built for head size {lib.attn_tc_head_dim()}, wanted {d}")
            self._attn_tc_libs[d] = lib
        return lib if lib.attn_prefill_tc_supports(page_size, nq, nkv) else None

    def _attention_library(self, d: int):
        lib = self._attn_libs.get(d)
        if lib is None:
            lib = build.load_library(f"attention_d{d}", ATTENTION_SOURCES, cuda=True, defines={"HEAD_DIM": d})
            lib.attn_decode_scratch_floats.restype = ctypes.c_size_t
            lib.attn_decode_flat_scratch_floats.restype = ctypes.c_size_t
            lib.kernels_set_pdl(1 if self.pdl else 0)
            if lib.attn_head_dim() != d:
                raise KernelError(f"attention library was built for head size {lib.attn_head_dim()}, wanted {d}")
            self._attn_libs[d] = lib
        return lib

    def decode_splits(self, S: int, nkv: int, max_context: int, blocks_per_sm: int = 2) -> int:
        """Splits of the key range per (request, key/value head) in a decode step.  Few requests:
        as many splits as keep all blocks resident at once, at most 8 (one cluster, which merges through its
        shared memory) and at least 256 keys each; a long context of very few requests takes more than 8 (at
        least 512 keys each, merged through scratch by the last block to arrive) when that at least doubles the
        blocks (one request of 32,768 keys: 43 -> 25 us a layer).  Many requests (more blocks than fit at
        once): the smallest count up to 4 whose last wave is at least 85 % as full as the best
        (the reference's heuristic has this shape, csrc/src/lib.rs:2122-2199)."""
        blocks = max(S * nkv, 1)
        capacity = self.num_sms * max(blocks_per_sm, 1)
        most = max(1, max_context // 256)
        if blocks < capacity:
            few = max(1, min(8, most, capacity // blocks))
            many = min(capacity // blocks, max_context // 512)
            return many if many >= 2 * few else few

        def efficiency(s):
            waves = blocks * s / capacity
            return waves / -(-blocks * s // capacity)

        most = min(most, 4)
        best = max(efficiency(s) for s in range(1, most + 1))
        return next(s for s in range(1, most + 1) if efficiency(s) >= 0.85 * best)

    def sample(self, logits, temperature, top_k, top_p, seed, step, out, num_rows=None, slots=None):
        """``slots`` (int32 per row): also leave each token in ``self.last_tokens[slot]`` for the next step."""
        R, V = logits.shape
        self._check(self.lib.sample_rows(_p(logits), R, V, _p(temperature), _p(top_k), _p(top_p), _p(seed), _p(step),
                                         _p(out), _p(num_rows), _p(slots), _p(self.last_tokens), self._stream()),
                    "sample_rows")

    def repeat_penalty(self, row, penalty: float, context):
        self._check(self.lib.repeat_penalty(_p(row), row.numel(), ctypes.c_float(penalty), _p(context),
                                            context.numel(), self._stream()), "repeat_penalty")
