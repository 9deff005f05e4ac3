"""FusedComm: tensor-parallel attention + expert-parallel MoE with the collectives fused into kernels.

The residual stream is *row-sharded* (sequence parallel): rank r owns rows [r*Tl, (r+1)*Tl) of the
step's T tokens.  Per layer:

  all-gather -> GEMM        the RMSNorm kernel of the owner quantises its rows to e4m3 and stores them
  (qkv_a, dense gate/up)    into every rank's gather buffer over NVLink; the consumer GEMM's TMA producer
                            waits per tile on the source rank's arrival flag, so tiles whose rows are
                            already here run while the rest are still in flight.
  GEMM -> reduce-scatter    the GEMM epilogue stores each partial output row (bf16) straight into the
  (o_proj, dense down)      owner's staging slot for this source; the owner's fused
                            sum + residual + RMSNorm + quant kernel waits for all sources.
  EP dispatch               router on own rows -> counts pushed to all ranks -> layout -> each token is
                            quantised once and stored at its expert-grouped row in the owner's receive
                            buffer together with its return address.
  grouped expert GEMMs      run on the receive buffer as soon as every source has signalled; the down
                            projection's epilogue stores each output row into the token owner's return
                            buffer (combine), where the weighted top-k sum (+ shared expert) is taken in
                            fixed k order.

Every wait is bounded; an expired wait raises the status word that ``ops._ext.check_status`` reads.
``NcclComm`` is the baseline implementing the same model-facing calls with NCCL collectives.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import _ext, fused as fused_ops, gemm as gemm_ops, moe as moe_ops
from ..ops.moe import ExpertWeights
from .comm import NcclComm
from .symm import MAX_WORLD, SymmetricHeap

FP8 = torch.float8_e4m3fn
AG_READY, RS_READY, CNT_READY, DISP_READY, RET_READY, A2A_READY = 0, 8, 16, 24, 32, 40
# rows this rank sends per step from which the gate/up grouped GEMM of the expert-parallel path runs on 128 x 256 tiles
WIDE_S1_MIN_ROWS = int(os.environ.get("BG_WIDE_S1_MIN_ROWS", "0"))
# rows this rank sends per step up to which the down-projection returns rows from the 128 x 256 kernel (per-thread
# 16-byte peer stores); larger steps keep the 128 x 128 kernel whose epilogue stages 128-byte runs through shared memory
WIDE_S3_MAX_ROWS = int(os.environ.get("BG_WIDE_S3_MAX_ROWS", "4096"))
ALIGN = 128


def _pad(n: int, a: int) -> int:
    return (n + a - 1) // a * a


class FusedComm(NcclComm):
    fused = True

    def __init__(self, device=None, group=None):
        super().__init__(group)
        self.device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        self.heap: Optional[SymmetricHeap] = None
        self.epoch = 0
        self.nvlink_bytes = 0
        self._started = False

    # ------------------------------------------------------------------ setup
    def configure(self, hidden: int, expert_hidden: int, num_experts: int, top_k: int, max_tokens: int,
                  a2a_bytes: int = 0) -> None:
        """Size and carve the symmetric heap for steps of at most ``max_tokens`` tokens (whole job).
        ``a2a_bytes``: capacity of each of the two all-to-all receive buffers (request-parallel attention)."""
        W = self.world
        T = _pad(max_tokens, W * 8)
        self.T_max, self.H, self.He, self.E, self.K = T, hidden, expert_hidden, num_experts, top_k
        Tl = T // W
        cap = _pad(T * top_k, ALIGN) + (num_experts // W) * ALIGN
        self.recv_cap = cap
        sizes = {
            "flags": 64 * 4,
            "ag_q": T * hidden, "ag_s": (hidden // 128) * _pad(T, 4) * 4,
            "rs_buf": T * hidden * 2,
            "cnt": W * num_experts * 4,
            "recv_q": cap * expert_hidden, "recv_s": (expert_hidden // 128) * _pad(cap, 4) * 4,
            "recv_info": cap * 8,
            "ret": Tl * top_k * expert_hidden * 2,
            "a2a0": _pad(a2a_bytes, 1024), "a2a1": _pad(a2a_bytes, 1024),
        }
        import os
        guard = 4096 if os.environ.get("BG_COMM_GUARD", "0") == "1" else 0    # debug: poisoned band after every region
        total = sum(_pad(v, 1024) + guard + 1024 for v in sizes.values()) + 64 * 1024
        self.heap = SymmetricHeap(total, self.device, self.group, guard_bytes=guard)
        for k, v in sizes.items():
            self.heap.alloc(k, v)
        h = self.heap
        # NVLS (opt-in, BG_NVLS=1): the broadcast pushes (normalised rows + scales of the all-gather, expert counts)
        # become one multimem store each instead of one store per peer
        self.nvls = os.environ.get("BG_NVLS", "0") == "1" and h.mc_base != 0
        L = _ext.lib()
        L.bg_comm_set_multicast.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
        with torch.cuda.device(self.device):
            if self.nvls:
                L.bg_comm_set_multicast(ctypes.c_void_p(h.mc_ptr("ag_q")), ctypes.c_void_p(h.mc_ptr("ag_s")),
                                        ctypes.c_void_p(h.mc_ptr("cnt")))
            else:
                L.bg_comm_set_multicast(None, None, None)
        self.flags = h.view("flags", torch.int32, (64,))
        self.flag_ptrs = h.peer_ptrs("flags")
        self.ag_q = h.view("ag_q", torch.uint8, (T, hidden)).view(FP8)
        self.ag_s_stride = _pad(T, 4)
        self.ag_s = h.view("ag_s", torch.float32, (hidden // 128, self.ag_s_stride))
        self.rs_buf = h.view("rs_buf", torch.bfloat16, (T, hidden))
        self.cnt = h.view("cnt", torch.int32, (W, num_experts))
        self.recv_q = h.view("recv_q", torch.uint8, (cap, expert_hidden)).view(FP8)
        self.recv_s_stride = _pad(cap, 4)
        self.recv_s = h.view("recv_s", torch.float32, (expert_hidden // 128, self.recv_s_stride))
        self.recv_info = h.view("recv_info", torch.int32, (cap, 2))
        self.ret = h.view("ret", torch.bfloat16, (Tl * top_k, expert_hidden))
        dev = self.device
        self.counters = torch.zeros(8, dtype=torch.int32, device=dev)
        self.row_base = torch.zeros(num_experts, dtype=torch.int32, device=dev)
        self.cursor = torch.zeros(num_experts, dtype=torch.int32, device=dev)
        El = num_experts // W
        self.offsets_buf = torch.zeros(2 * El + 1, dtype=torch.int32, device=dev)   # [El + 1 offsets | El real counts]
        self.offsets = self.offsets_buf[: El + 1]
        self.recv_counts = self.offsets_buf[El + 1:]
        self.total_rows = torch.zeros(1, dtype=torch.int32, device=dev)
        self.sent_row = torch.zeros(Tl * top_k, dtype=torch.int32, device=dev)
        self.ident_pos = torch.arange(Tl * top_k, dtype=torch.int32, device=dev)
        self.a2a_bytes = _pad(a2a_bytes, 1024)
        self.a2a_bufs = [h.view("a2a0", torch.uint8, (self.a2a_bytes,)), h.view("a2a1", torch.uint8, (self.a2a_bytes,))] \
            if a2a_bytes else []
        self._a2a_turn = 0
        self.last = {AG_READY: 0, RS_READY: 0, CNT_READY: 0, DISP_READY: 0, RET_READY: 0, A2A_READY: 0}
        # Epochs are (offset within the step) + (device-resident base).  The base is bumped by a kernel at
        # the end of every step, so a captured CUDA graph advances its epochs on every replay.
        self.epoch_base = torch.zeros(1, dtype=torch.int32, device=dev)
        self.epoch = 0
        self.heap.barrier()

    def begin_step(self) -> None:
        if not self._started:
            # the first step's kernels wait on peers with a bounded budget: start it together (ranks finish
            # loading weights at different times)
            self._started = True
            if not torch.cuda.is_current_stream_capturing():
                self.heap.barrier()
        self.epoch = 0
        for k in self.last:
            self.last[k] = 0

    def end_step(self) -> None:
        """Advance the device epoch base past every epoch this step used (stream-ordered)."""
        rc = _ext.lib().bg_bump_epoch(_ext.ptr(self.epoch_base), ctypes.c_uint32(self.epoch), _ext.stream())
        _ext.check(rc, "bg_bump_epoch")
        self.epoch = 0

    def _next(self, kind: int) -> int:
        self.epoch += 1
        self.last[kind] = self.epoch
        return self.epoch

    def _base(self):
        return _ext.ptr(self.epoch_base)

    def _flag_ptr(self, kind: int):
        return ctypes.c_void_p(self.flags.data_ptr() + 4 * kind)

    def _status(self):
        return _ext.ptr(_ext.status_word(self.device))

    # ------------------------------------------------------------------ sequence-parallel primitives
    def sp_norm_push(self, src: Optional[torch.Tensor], residual: torch.Tensor, weight: torch.Tensor, eps: float,
                     from_rs: bool, has_residual: bool, push: bool, want_y: bool = True, want_q: bool = True):
        """Owner-side fused (sum of reduce-scatter partials | local rows) + residual + RMSNorm + quant,
        optionally pushing the quantised rows into every rank's gather buffer.
        Returns (y bf16 | None, q | None, s | None) for the rank's own rows."""
        W, Tl = self.world, residual.shape[0]
        H = residual.shape[1]
        dev = self.device
        y = torch.empty(Tl, H, dtype=torch.bfloat16, device=dev) if want_y else None
        q = s = None
        s_stride = 0
        if want_q:
            q = torch.empty(Tl, H, dtype=FP8, device=dev)
            s = fused_ops._scale_buffer(Tl, H // 128, dev)
            s_stride = s.stride(1)
        if from_rs:
            partials, n_src = self.rs_buf, W
            ready, wait_epoch = self._flag_ptr(RS_READY), self.last[RS_READY]
        else:
            partials, n_src = src, 1
            ready, wait_epoch = ctypes.c_void_p(0), 0
        epoch = self._next(AG_READY) if push else 0
        rc = _ext.lib().bg_sp_norm_quant_push(
            _ext.ptr(partials), ctypes.c_int(n_src), ready, ctypes.c_uint32(wait_epoch), self._base(),
            _ext.ptr(residual),
            ctypes.c_int(int(has_residual)), _ext.ptr(weight), _ext.ptr(y), _ext.ptr(q), _ext.ptr(s),
            ctypes.c_int(s_stride), self.heap.peer_ptrs("ag_q"), self.heap.peer_ptrs("ag_s"),
            ctypes.c_int(self.ag_s_stride), ctypes.c_int(int(push)), ctypes.c_int(Tl), ctypes.c_int(H),
            ctypes.c_float(eps), ctypes.c_int(self.rank), ctypes.c_int(W), self.flag_ptrs, ctypes.c_int(AG_READY),
            ctypes.c_uint32(epoch), _ext.ptr(self.counters[0:1]), self._status(), _ext.stream())
        _ext.check(rc, "bg_sp_norm_quant_push")
        if push:
            self.nvlink_bytes += (W - 1) * Tl * (H + 4 * (H // 128))
        return y, q, s

    def _set_hooks(self, a_ready=None, a_ready_rows=0, epoch=0, m_rotate=0, peer_out=None, row_map=None,
                   rs_rows=0, done_index=0, done_counter=None, peer_flags=None):
        gemm_ops.hooks_pending()                 # the next GEMM consumes these hooks on the 128 x 128 kernel
        _ext.lib().bg_gemm_set_hooks(
            a_ready if a_ready is not None else ctypes.c_void_p(0), ctypes.c_int(a_ready_rows), ctypes.c_uint32(epoch),
            self._base(), ctypes.c_int(m_rotate), peer_out if peer_out is not None else ctypes.c_void_p(0),
            _ext.ptr(row_map), ctypes.c_int(rs_rows), ctypes.c_int(self.rank), ctypes.c_int(self.world),
            peer_flags if peer_flags is not None else ctypes.c_void_p(0), ctypes.c_int(done_index),
            _ext.ptr(done_counter))

    def ag_gemm(self, lin, T: int, silu_mul: bool = False) -> torch.Tensor:
        """[T, K] (gathered e4m3 rows in the symmetric buffer) x W^T; tiles start as their source
        rank's rows arrive, this rank's own rows first."""
        Tl = T // self.world
        tiles_per_rank = max(1, Tl // 128)
        self._set_hooks(a_ready=self._flag_ptr(AG_READY), a_ready_rows=Tl, epoch=self.last[AG_READY],
                        m_rotate=(self.rank * Tl) // 128 if Tl % 128 == 0 else 0)
        xs = self.ag_s.t()[:T]
        return gemm_ops.fp8_gemm(self.ag_q[:T], xs, lin.w, lin.s, silu_mul=silu_mul and lin.interleaved)

    def gemm_rs(self, xq, xs, lin, T: int) -> None:
        """Partial GEMM [T, Kshard] x W^T whose epilogue stores every output row into its owner's
        staging slot for this rank; remote rows are computed first."""
        Tl = T // self.world
        epoch = self._next(RS_READY)
        rot = (((self.rank + 1) % self.world) * Tl) // 128 if Tl % 128 == 0 else 0
        self._set_hooks(m_rotate=rot, peer_out=self.heap.peer_ptrs("rs_buf"), rs_rows=Tl, epoch=epoch,
                        done_index=RS_READY, done_counter=self.counters[1:2], peer_flags=self.flag_ptrs)
        N = lin.w.shape[0]
        out = self.rs_buf.view(-1)[: T * N].view(T, N)      # only its row stride is used by the scatter epilogue
        gemm_ops.fp8_gemm(xq, xs, lin.w, lin.s, out=out)
        self.nvlink_bytes += (self.world - 1) * Tl * N * 2

    # ------------------------------------------------------------------ all-to-all over peer memory
    def all_to_all(self, x: torch.Tensor) -> torch.Tensor:
        """x [world, ...]: slice d is stored into rank d's receive buffer by a push kernel (plain peer stores +
        arrival flags), then a one-warp kernel waits for every rank's flag.  Two receive buffers alternate, so a
        result stays valid until the call after next.  Falls back to NCCL for messages beyond the buffers."""
        W = self.world
        x = x.contiguous()
        nbytes = x.numel() * x.element_size()
        slice_bytes = nbytes // W
        if W == 1 or not self.a2a_bufs or nbytes > self.a2a_bytes or slice_bytes % 16:
            return super().all_to_all(x)
        buf = self._a2a_exchange(x, 1, slice_bytes, slice_bytes, 0, slice_bytes, 0)
        return buf[:nbytes].view(x.dtype).view(x.shape)

    def _a2a_exchange(self, x, n_chunks, chunk_bytes, src_d, src_b, dst_r, dst_b) -> torch.Tensor:
        """One chunked push (see ``a2a_push_kernel``) plus the wait for every rank's arrival flag; returns the
        receive buffer (bytes)."""
        W = self.world
        name = "a2a0" if self._a2a_turn == 0 else "a2a1"
        buf = self.a2a_bufs[self._a2a_turn]
        self._a2a_turn ^= 1
        epoch = self._next(A2A_READY)
        st = _ext.stream()
        ull = ctypes.c_ulonglong
        rc = _ext.lib().bg_a2a_push_chunks(_ext.ptr(x), self.heap.peer_ptrs(name), ull(n_chunks), ull(chunk_bytes),
                                           ull(src_d), ull(src_b), ull(dst_r), ull(dst_b), ctypes.c_int(self.rank),
                                           ctypes.c_int(W), self.flag_ptrs, ctypes.c_int(A2A_READY),
                                           ctypes.c_uint32(epoch), self._base(), _ext.ptr(self.counters[4:5]), st)
        _ext.check(rc, "bg_a2a_push_chunks")
        rc = _ext.lib().bg_wait_flags(self._flag_ptr(A2A_READY), ctypes.c_int(W), ctypes.c_uint32(epoch), self._base(),
                                      self._status(), st)
        _ext.check(rc, "bg_wait_flags")
        self.nvlink_bytes += n_chunks * chunk_bytes * (W - 1)
        return buf

    def _a2a_fits(self, x: torch.Tensor, chunk_bytes: int) -> bool:
        return (self.world > 1 and bool(self.a2a_bufs) and x.is_contiguous()
                and x.numel() * x.element_size() <= self.a2a_bytes and chunk_bytes % 16 == 0)

    def a2a_rows_to_ranks(self, x: torch.Tensor) -> torch.Tensor:
        """[world * n, c] -> [n, world, c]; the push kernel stores each row's piece at its final place, so no
        transposing copy follows."""
        W = self.world
        n, c = x.shape[0] // W, x.shape[1]
        cb = c * x.element_size()
        if not self._a2a_fits(x, cb):
            return super().a2a_rows_to_ranks(x)
        buf = self._a2a_exchange(x, n, cb, n * cb, cb, cb, W * cb)
        return buf[: x.numel() * x.element_size()].view(x.dtype).view(n, W, c)

    def a2a_ranks_to_rows(self, x: torch.Tensor) -> torch.Tensor:
        """[n, world, c] -> [world * n, c], reading each destination's pieces in place."""
        n, W, c = x.shape
        cb = c * x.element_size()
        if not self._a2a_fits(x, cb):
            return super().a2a_ranks_to_rows(x)
        buf = self._a2a_exchange(x, n, cb, cb, W * cb, n * cb, cb)
        return buf[: x.numel() * x.element_size()].view(x.dtype).view(W * n, c)

    # ------------------------------------------------------------------ expert parallel
    def moe_sp(self, h_local: torch.Tensor, topk_idx: torch.Tensor, topk_w: torch.Tensor, ew: ExpertWeights,
               extra: Optional[torch.Tensor] = None, timer=None, before_combine=None) -> torch.Tensor:
        """Routed-expert output for this rank's own rows (dispatch -> experts -> combine).  ``before_combine`` is
        called right before the combine reads ``extra`` (the caller may have computed it on another stream)."""
        if timer is None:
            from ..utils.timing import null_timer
            timer = null_timer()
        W, E, K = self.world, self.E, topk_idx.shape[1]
        Tl, H = h_local.shape
        L = _ext.lib()
        st = _ext.stream()
        # decode-sized steps (about one 32-token tile per expert): weights on the MMA's M side, segments aligned to
        # the 32-token tile so that the padded row count stays close to the real one
        small = gemm_ops.use_swapab(Tl * K / max(E // W, 1), ew.w13.shape[1], ew.w13.shape[2]) and \
            ew.w2.shape[1] % 128 == 0 and ew.w2.shape[2] % 128 == 0
        align = 32 if small else ALIGN
        with timer.timed("moe.ep_count_layout"):
            e_cnt = self._next(CNT_READY)
            rc = L.bg_ep_count_push(_ext.ptr(topk_idx), ctypes.c_int(Tl * K), ctypes.c_int(E),
                                    self.heap.peer_ptrs("cnt"), ctypes.c_int(self.rank), ctypes.c_int(W),
                                    self.flag_ptrs, ctypes.c_int(CNT_READY), ctypes.c_uint32(e_cnt), self._base(),
                                    _ext.ptr(self.recv_info),
                                    ctypes.c_int(min(self.recv_cap, _pad(W * Tl * K, align) + (E // W) * align)), st)
            _ext.check(rc, "bg_ep_count_push")
            rc = L.bg_ep_layout(_ext.ptr(self.cnt), self._flag_ptr(CNT_READY), ctypes.c_uint32(e_cnt), self._base(),
                                ctypes.c_int(E), ctypes.c_int(W), ctypes.c_int(self.rank), ctypes.c_int(align),
                                _ext.ptr(self.row_base), _ext.ptr(self.offsets), _ext.ptr(self.cursor),
                                _ext.ptr(self.total_rows), self._status(), st)
            _ext.check(rc, "bg_ep_layout")
        with timer.timed("moe.ep_dispatch"):
            e_disp = self._next(DISP_READY)
            rc = L.bg_ep_dispatch_send(_ext.ptr(h_local), ctypes.c_int(h_local.stride(0)), _ext.ptr(topk_idx),
                                       ctypes.c_int(Tl), ctypes.c_int(K), ctypes.c_int(E), ctypes.c_int(H),
                                       _ext.ptr(self.row_base), _ext.ptr(self.cursor), self.heap.peer_ptrs("recv_q"),
                                       self.heap.peer_ptrs("recv_s"), ctypes.c_int(self.recv_s_stride),
                                       self.heap.peer_ptrs("recv_info"), ctypes.c_int(self.recv_cap),
                                       _ext.ptr(self.sent_row), ctypes.c_int(self.rank), ctypes.c_int(W), self.flag_ptrs,
                                       ctypes.c_int(DISP_READY), ctypes.c_uint32(e_disp), self._base(),
                                       _ext.ptr(self.counters[2:3]),
                                       self._status(), st)
            _ext.check(rc, "bg_ep_dispatch_send")
        self.nvlink_bytes += Tl * K * (H + 4 * (H // 128)) * (W - 1) // W
        # ---- experts on the receive buffer: the gate/up GEMM waits for every source rank's rows
        xs = self.recv_s.t()[: self.recv_cap]
        if timer.enabled:
            # profiling only: take the wait for the peers' rows out of the GEMM's interval
            with timer.timed("moe.dispatch_wait"):
                _ext.check(L.bg_wait_flags(self._flag_ptr(DISP_READY), ctypes.c_int(W), ctypes.c_uint32(e_disp),
                                           self._base(), self._status(), st), "bg_wait_flags")
        with timer.timed("moe.s1_gemm"):
            if small:
                act = gemm_ops.grouped_fp8_gemm(self.recv_q, xs, ew.w13, ew.w13_s, self.offsets, silu_mul=True,
                                                counts=self.recv_counts, rows_hint=Tl * K,
                                                a_ready=(self._flag_ptr(DISP_READY), e_disp, self._base(), W))
            elif gemm_ops.wide_enabled() and Tl * K >= WIDE_S1_MIN_ROWS:
                # prefill-sized steps: 128 x 256 tiles (less operand traffic per FLOP); its producer waits for
                # the arrival flags itself
                act = gemm_ops.grouped_fp8_gemm(self.recv_q, xs, ew.w13, ew.w13_s, self.offsets, silu_mul=True,
                                                counts=self.recv_counts,
                                                a_ready=(self._flag_ptr(DISP_READY), e_disp, self._base(), W))
            else:
                self._set_hooks(a_ready=self._flag_ptr(DISP_READY), a_ready_rows=0, epoch=e_disp)
                act = gemm_ops.grouped_fp8_gemm(self.recv_q, xs, ew.w13, ew.w13_s, self.offsets, silu_mul=True,
                                                counts=self.recv_counts)
        with timer.timed("moe.act_quant"):
            # one block per row: launch over the rows this step can have received (every rank's rows x top-k plus
            # one alignment gap per local expert), not over the whole receive capacity sized for prefill steps
            bound = min(self.recv_cap, _pad(W * Tl * K, align) + (E // W) * align)
            aq, as_ = fused_ops.act_quant(act[:bound], valid_rows=self.total_rows)
        # ---- down projection; the epilogue returns each row to its token's owner (combine)
        with timer.timed("moe.s3_gemm_return"):
            e_ret = self._next(RET_READY)
            El, Hout, I = ew.w2.shape
            if small:
                sc, sc_stride = gemm_ops._scales_kb_major(as_)
                rc = L.bg_gemm_fp8_swapab_return(
                    _ext.ptr(aq), _ext.ptr(sc), ctypes.c_int(sc_stride), _ext.ptr(ew.w2), _ext.ptr(ew.w2_s),
                    ctypes.c_int(Hout), _ext.ptr(self.offsets), _ext.ptr(self.recv_counts), ctypes.c_int(El),
                    ctypes.c_int(aq.shape[0]), ctypes.c_int(Hout), ctypes.c_int(I), ctypes.c_int(_ext.num_sms(self.device)),
                    self.heap.peer_ptrs("ret"), _ext.ptr(self.recv_info), self.flag_ptrs, ctypes.c_int(RET_READY),
                    ctypes.c_uint32(e_ret), self._base(), _ext.ptr(self.counters[3:4]), ctypes.c_int(self.rank),
                    ctypes.c_int(W), self._status(), st)
                _ext.check(rc, "bg_gemm_fp8_swapab_return")
            elif gemm_ops.wide_enabled() and Tl * K <= WIDE_S3_MAX_ROWS and Hout % 8 == 0 and I % 128 == 0:
                # decode-sized steps: 128 x 256 tiles stream the weights faster; rows leave with plain 16-byte stores
                sc, sc_stride = gemm_ops._scales_kb_major(as_)
                rc = L.bg_gemm_fp8_n256_return(
                    _ext.ptr(aq), _ext.ptr(sc), ctypes.c_int(sc_stride), _ext.ptr(ew.w2), _ext.ptr(ew.w2_s),
                    ctypes.c_int(Hout), _ext.ptr(self.offsets), _ext.ptr(self.recv_counts), ctypes.c_int(El),
                    ctypes.c_int(aq.shape[0]), ctypes.c_int(Hout), ctypes.c_int(I), ctypes.c_int(_ext.num_sms(self.device)),
                    self.heap.peer_ptrs("ret"), _ext.ptr(self.recv_info), self.flag_ptrs, ctypes.c_int(RET_READY),
                    ctypes.c_uint32(e_ret), self._base(), _ext.ptr(self.counters[3:4]), ctypes.c_int(self.rank),
                    ctypes.c_int(W), self._status(), st)
                _ext.check(rc, "bg_gemm_fp8_n256_return")
            else:
                self._set_hooks(peer_out=self.heap.peer_ptrs("ret"), row_map=self.recv_info, epoch=e_ret,
                                done_index=RET_READY, done_counter=self.counters[3:4], peer_flags=self.flag_ptrs)
                out_stub = self.rs_buf.view(-1)[: ew.w2.shape[1]].view(1, -1)   # row stride carrier only
                gemm_ops.grouped_fp8_gemm(aq, as_, ew.w2, ew.w2_s, self.offsets,
                                          out=_StrideCarrier(out_stub, self.recv_cap), counts=self.recv_counts)
        self.nvlink_bytes += Tl * K * H * 2 * (W - 1) // W
        with timer.timed("moe.return_wait_combine"):
            rc = L.bg_wait_flags(self._flag_ptr(RET_READY), ctypes.c_int(W), ctypes.c_uint32(e_ret), self._base(),
                                 self._status(), st)
            _ext.check(rc, "bg_wait_flags")
            if before_combine is not None:
                before_combine()
            return moe_ops.combine(self.ret[: Tl * K], self.ident_pos[: Tl * K].view(Tl, K), topk_w, extra)


class _StrideCarrier:
    """Stands in for an output tensor when the GEMM's scatter epilogue stores rows into peer memory:
    only ``stride(0)``, ``data_ptr`` and ``shape`` are consulted by the launcher."""

    def __init__(self, row: torch.Tensor, rows: int):
        self._row, self.shape = row, (rows, row.shape[1])

    def stride(self, i: int) -> int:
        return self._row.shape[1] if i == 0 else 1

    def data_ptr(self) -> int:
        return self._row.data_ptr()


def bounded_flag_wait(flags: torch.Tensor, n: int, epoch: int, budget_ms: int) -> None:
    """Enqueue a wait until ``flags[i] >= epoch`` for i < n (``flags``: int32 device tensor) that gives up
    after ``budget_ms`` and raises the device status word instead of hanging; read the outcome with
    ``ops._ext.check_status``.  Used by the failure-detection tests and by health probes of a peer."""
    rc = _ext.lib().bg_wait_flags_budget(_ext.ptr(flags), ctypes.c_int(n), ctypes.c_uint32(epoch), ctypes.c_void_p(0),
                                         ctypes.c_int(budget_ms), _ext.ptr(_ext.status_word(flags.device)),
                                         _ext.stream())
    _ext.check(rc, "bg_wait_flags_budget")
