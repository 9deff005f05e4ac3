"""The batch engine: one scheduling loop per rank that alternates prefill waves and decode
intervals until every admitted sequence completes.

Design (B200-first; differs from the reference on purpose): with 180 GB of HBM per GPU the *device*
page pool is the primary KV store — prefill writes latent KV straight into GPU pages and decode reads
them in place — and the pinned host tier is the overflow: rows put ON_HOLD at a page boundary are
copied out on a side stream, loaded back when space frees up, and rows whose KV cannot be kept
anywhere are EVICTED and recomputed.  The reference is host-KV-first (prefill offloads every layer's
KV to CPU DRAM and decode streams it back, batchgen/batchgen_worker.py:6491-7290); the scheduling
*policy* (admission order, marginal page charges, boundary decisions every ``decision_interval``
decode tokens, watermark re-entry into prefill) is kept, see ``scheduler.py``.

All ranks of a TP/EP job run this loop in lock step over identical inputs, so every decision is taken
redundantly and identically on each rank; only model collectives cross ranks.

Two model paths sit under the same loop.  With the NCCL baseline (or one GPU) every rank calls
``Transformer.forward`` on all rows of the step and samples all of them identically.  With the fused
NVLink kernels (``parallel.fused.FusedComm`` and a sequence-parallel weight layout) the step is padded to a
multiple of the world size, every rank calls ``Transformer.forward_sp`` and receives the logits of its own
block of rows only, samples those, and the sampled tokens are all-gathered (``_sample_sharded``), so that
every rank again holds every token before the next scheduling decision.
"""
from __future__ import annotations

import time
from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence as Seq

import torch

from ..config import EngineConfig, ModelConfig
from ..models.transformer import AttnMeta, Transformer
from ..ops import sampling as sampling_ops
from . import scheduler as sched
from . import trajectory as trajectory_mod
from . import wave_plan
from .kv_cache import HostStateStore, PagedKVCache, build_block_table, slots_for_range
from .prefix_cache import PrefixCache
from .sequence import (PageBufferConfig, SamplingParams, Sequence, SequenceStatus, gpu_pages_first_load,
                       pages_for)

S = SequenceStatus


@dataclass
class _PrefillRow:
    """One packed row of a prefill micro-batch: ``tokens`` continue a context of ``start`` tokens whose KV sits in
    the first pages of ``pages`` (``pages`` covers positions 0 .. start + len(tokens)).  ``seq`` receives the token
    sampled from the row's last position; rows without a sequence (a shared prefix computed once for several
    prompts) produce no logits.  ``state_slot`` names the per-sequence state (recurrent or window / compressor state)
    the row advances: every piece of a chunked prompt carries it, although only the last piece has ``seq``."""
    tokens: List[int]
    start: int
    pages: List[int]
    seq: Optional[Sequence] = None
    state_slot: int = -1

    def __post_init__(self):
        if self.seq is not None and self.state_slot < 0:
            self.state_slot = self.seq.state_slot


@dataclass
class EngineStats:
    prefill_tokens: int = 0
    prefill_cached_tokens: int = 0
    prefill_seconds: float = 0.0
    decode_tokens: int = 0
    decode_seconds: float = 0.0
    decode_steps: int = 0
    prefill_waves: int = 0
    holds: int = 0
    evictions: int = 0
    loads: int = 0
    offloaded_pages: int = 0
    shared_prefix_tokens: int = 0      # prompt tokens not computed because another prompt of the wave shares them
    trajectory_commits: int = 0        # completed rows whose prompt + output pages were left in the prefix cache
    prefill_chunks: int = 0            # forwards that computed a piece of a prompt longer than max_prefill_tokens
    growth_evictions: int = 0          # parked rows evicted to make host-tier room for a row that had to be parked
    transfer_waits: int = 0            # times the host blocked on a page transfer (pool exhausted with copies in flight)
    trajectory_frontiers: int = 0      # finished turns of sessions whose pages were pinned as the session's frontier
    trajectory_restores: int = 0       # turns that extended their session's frontier
    prefix_promoted_pages: int = 0     # prefix pages brought back from the host tier's coordinator

    def summary(self) -> Dict[str, float]:
        return dict(
            prefill_tok_per_s=self.prefill_tokens / self.prefill_seconds if self.prefill_seconds else 0.0,
            decode_tok_per_s=self.decode_tokens / self.decode_seconds if self.decode_seconds else 0.0,
            **self.__dict__)


class Engine:
    def __init__(self, model: Transformer, ecfg: EngineConfig, num_gpu_pages: Optional[int] = None,
                 num_host_pages: int = 0, on_complete: Optional[Callable[[Sequence], None]] = None,
                 graph_runner=None, host_kv_fd: Optional[int] = None):
        ecfg.validate()
        self.model, self.cfg, self.ecfg = model, model.cfg, ecfg
        self.device = model.device
        self.buf = PageBufferConfig(ecfg.page_size, ecfg.initial_gpu_page_buffer, ecfg.extension_gpu_page_buffer,
                                    ecfg.decision_frequency_pages)
        kv_dtype = model.dtype
        n_pages = num_gpu_pages or ecfg.num_gpu_pages
        if not n_pages:
            raise ValueError("num_gpu_pages must be given (see planner.size_kv_pool for automatic sizing)")
        state_slots, state_heads = 0, None
        if self.cfg.has_kda:
            # every live sequence holds one recurrent-state slot from its prefill until it completes or is evicted
            state_slots = ecfg.max_state_slots or ecfg.max_decode_batch
            state_heads = next(lw.kda.heads for lw in model.w.layers if lw.kda is not None)
            if ecfg.enable_prefix_cache:
                raise ValueError("prefix reuse needs per-page state snapshots, which KDA layers do not keep")
        elif self.cfg.is_v4:
            # every live sequence holds one slot of window rings and compressor windows
            state_slots = ecfg.max_state_slots or ecfg.max_decode_batch
            if ecfg.enable_prefix_cache:
                raise ValueError("prefix reuse needs per-page snapshots of the window and compressor state, which "
                                 "DeepSeek-V4 layers do not keep")
        self.kv = PagedKVCache(self.cfg, n_pages, ecfg.page_size, self.device, kv_dtype, state_slots=state_slots,
                               state_heads=state_heads)
        # host tier: on a GPU the native region + asynchronous movers (a region created by the server is attached
        # through ``host_kv_fd``); the pinned torch tensor is the CPU / fallback form of the same tier
        self.host_tier = None
        if (num_host_pages or host_kv_fd is not None) and self.device.type == "cuda" \
                and ecfg.host_kv_backend == "native" and not self.cfg.has_kda and not self.cfg.is_v4:
            from .host_tier import NativeHostTier
            self.host_tier = NativeHostTier(self.kv, num_host_pages, fd=host_kv_fd)
            self.host_kv = self.host_tier                  # same allocator face (``.alloc``)
        else:
            self.host_kv = (PagedKVCache(self.cfg, num_host_pages, ecfg.page_size, "cpu", kv_dtype, pinned=True)
                            if num_host_pages else None)
        from .continuous_batching import AdaptiveChunkSizer
        # host-KV reservation chunk follows the decode lengths actually seen (EMA), from the configured start value
        self.chunk_sizer = AdaptiveChunkSizer(initial_chunk=ecfg.host_kv_chunk_size,
                                              min_chunk=min(ecfg.adaptive_chunk_min, ecfg.host_kv_chunk_size),
                                              max_chunk=max(ecfg.adaptive_chunk_max, ecfg.host_kv_chunk_size),
                                              ema_alpha=ecfg.adaptive_chunk_ema_alpha,
                                              multiplier=ecfg.adaptive_chunk_multiplier)
        from ..utils.step_ring import StepRing
        self.step_ring = StepRing(256)                     # the most recent forwards, for heartbeats and fatal messages
        self._deferred_gpu: List[tuple] = []               # (transfer tasks, device pages freed when they are done)
        self._deferred_host: List[tuple] = []              # (transfer tasks, host pages released when they are done)
        self.host_state = None
        if self.kv.state is not None and self.host_kv is not None:
            self.host_state = HostStateStore(self.kv.state, ecfg.max_host_state_items or 4 * state_slots)
        self.prefix = PrefixCache(self.kv.alloc, ecfg.page_size) if ecfg.enable_prefix_cache else None
        # session frontiers: the pages of a session's last finished turn hold an extra reference, so cache pressure
        # from other requests cannot evict a live conversation's context (released by end_session, by a diverging
        # prompt, or oldest first when the pool runs short)
        self.trajectories = None
        self._session_lru: "OrderedDict[str, None]" = OrderedDict()
        if self.prefix is not None:
            self.trajectories = trajectory_mod.TrajectoryFrontierRegistry(
                ecfg.page_size, self.kv.bytes_per_page(),
                release_fn=lambda rec: self.kv.alloc.free(list(rec.page_ids)))
        self.kv_token_budget = (ecfg.max_model_len if ecfg.max_model_len > 0 else n_pages * ecfg.page_size)
        self.seqs: Dict[int, Sequence] = {}
        self._next_idx = 0
        self.stats = EngineStats()
        self.on_complete = on_complete
        self.graph_runner = graph_runner
        self.copy_stream = torch.cuda.Stream() if self.device.type == "cuda" else None
        self.guard = sched.PrefillProgressGuard()
        self._gen = torch.Generator(device=self.device)
        self._gen.manual_seed(ecfg.seed)
        self.step_hook: Optional[Callable[[str], None]] = None   # watchdog feed
        comm = model.comm
        # > 1: the model runs forward_sp over a row-sharded residual stream (fused NVLink kernels)
        self.sp_world = (comm.world if (comm is not None and getattr(comm, "fused", False) and comm.world > 1
                                        and model.layout.sequence_parallel) else 1)
        from .sampling_residency import DecodeSamplingResidency
        self._residency = DecodeSamplingResidency(max(ecfg.max_decode_batch, 1) + 8 * max(self.sp_world, 1),
                                                  self.device)
        self._samp_key: Optional[tuple] = None
        self._samp_rows: List[Optional[Sequence]] = []
        self._samp_epoch = 0

    # ------------------------------------------------------------------ intake
    def add_request(self, prompt_ids: Seq[int], params: Optional[SamplingParams] = None, custom_id: str = "",
                    batch_id: str = "", prefill_order: Optional[int] = None,
                    session_id: Optional[str] = None) -> Sequence:
        if len(prompt_ids) == 0:
            raise ValueError("empty prompt")
        params = params or SamplingParams()
        if self.ecfg.max_model_len > 0 and len(prompt_ids) + params.max_new_tokens > self.ecfg.max_model_len:
            raise ValueError(f"context {len(prompt_ids)} + {params.max_new_tokens} exceeds max_model_len "
                             f"{self.ecfg.max_model_len}")
        s = Sequence(global_idx=self._next_idx, prompt_ids=list(map(int, prompt_ids)), params=params,
                     custom_id=custom_id, batch_id=batch_id, prefill_order=prefill_order)
        self._next_idx += 1
        self.seqs[s.global_idx] = s
        if session_id and self.trajectories is not None:
            s.session_id = session_id
            # the session's committed frontier: a hit means the turn extends it (its pages come back through the
            # prefix cache, pinned until now by the frontier); a prompt that diverges makes the frontier useless
            res = self.trajectories.resolve(session_id, s.prompt_ids)
            if res.hit:
                self.stats.trajectory_restores += 1
                res.record.release()                    # the sequence takes its own page references at prefill
            elif res.reason == trajectory_mod.DECLINE_PROMPT_DIVERGES:
                self.end_session(session_id)
        return s

    def end_session(self, session_id: str) -> bool:
        """Drop the session's frontier (its pages go back to being ordinary prefix-cache entries)."""
        if self.trajectories is None or self.trajectories.get(session_id) is None:
            return False
        self.trajectories.evict(session_id)
        self._session_lru.pop(session_id, None)
        return True

    def adopt_sequence(self, prompt_ids: Seq[int], output_ids: Seq[int], params: Optional[SamplingParams] = None,
                       custom_id: str = "", batch_id: str = "", gpu_pages: Optional[List[int]] = None) -> Sequence:
        """Register a sequence whose KV already sits in device pages: a restored trajectory, a row received from
        another rank, or a benchmark's synthetic context.  ``output_ids`` must hold at least the first generated
        token (the next decode step feeds the last one).  Pages are allocated here unless ``gpu_pages`` (already
        owned by the caller through ``self.kv.alloc``) is given; the row enters as PREFILLED."""
        if not output_ids:
            raise ValueError("an adopted sequence carries at least its first generated token")
        s = Sequence(global_idx=self._next_idx, prompt_ids=list(map(int, prompt_ids)),
                     params=params or SamplingParams(), custom_id=custom_id, batch_id=batch_id)
        s.output_ids = list(map(int, output_ids))
        s.num_cached_tokens = s.context_len - 1
        need = pages_for(s.context_len, self.buf.page_size)
        if gpu_pages is None:
            gpu_pages = self._take_pages(need)
        elif len(gpu_pages) < need:
            raise ValueError(f"{len(gpu_pages)} pages given, the context needs {need}")
        s.gpu_pages = list(gpu_pages)
        s.status = S.PREFILLED
        s.history.append("adopted")
        self._next_idx += 1
        self.seqs[s.global_idx] = s
        return s

    def decode_steps(self, max_steps: int) -> int:
        """Admit decodable rows and decode at most ``max_steps`` tokens per row (a decode interval cut short),
        then apply the boundary decisions.  Returns the steps executed."""
        return self._decode_interval(max_steps=max_steps)

    # ------------------------------------------------------------------ helpers
    def _by_status(self, *st) -> List[Sequence]:
        return [s for s in self.seqs.values() if s.status in st]

    def _free_pages(self) -> int:
        """Device pages available to the scheduler: free ones plus those whose offload is still in flight (they are
        free by the time anything is written to them, see ``_take_pages``).  Counting them makes the schedule
        independent of transfer timing."""
        if self._deferred_gpu or self._deferred_host:
            self._drain_deferred()
        return self.kv.alloc.num_free + sum(len(p) for _, p in self._deferred_gpu)

    def _take_pages(self, n: int) -> List[int]:
        """Allocate device pages; blocks on transfers in flight only when the free list alone cannot serve."""
        if self._deferred_gpu and self.kv.alloc.num_free < n:
            self._drain_deferred()
            if self.kv.alloc.num_free < n:
                self._drain_deferred(block=True)
        return self.kv.alloc.alloc(n)

    def _drain_deferred(self, block: bool = False) -> None:
        """Pages that a transfer in flight still reads go back to their allocator once the transfer is done."""
        if self.host_tier is None:
            return
        for queue, alloc in ((self._deferred_gpu, self.kv.alloc), (self._deferred_host, self.host_tier.alloc)):
            keep = []
            for tasks, pages in queue:
                if block:
                    self.host_tier.wait(tasks)
                    self.stats.transfer_waits += 1
                if block or self.host_tier.done(tasks):
                    alloc.free(pages)
                else:
                    keep.append((tasks, pages))
            queue[:] = keep

    def _sync(self) -> None:
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)

    def _reclaim(self, want: int) -> int:
        if want <= 0:
            return 0
        if self.prefix is None:
            return 0
        # demoted pages count as free at once (``_free_pages``); ``_take_pages`` waits for their copies if it must
        on_evict = self._demote_prefix_page if self.host_tier else None
        got = self.prefix.evict(want, on_evict=on_evict)
        if got < want and self.trajectories is not None and len(self.trajectories):
            # still short: the oldest idle sessions give up their pins, then the cache can let those pages go
            if self.trajectories.evict_for_pages(want - got, list(self._session_lru)):
                for sid in [k for k in self._session_lru if self.trajectories.get(k) is None]:
                    self._session_lru.pop(sid, None)
                got += self.prefix.evict(want - got, on_evict=on_evict)
        return got

    def _demote_prefix_page(self, key: bytes, page: int) -> bool:
        """A prefix page leaves the device cache: keep it in the host tier's coordinator.  Returns True when the
        page's release was taken over (it is freed when the copy is done)."""
        stream = torch.cuda.current_stream().cuda_stream
        tasks = self.host_tier.demote(key, page, after_stream=stream)
        if tasks is None:
            return False
        self._deferred_gpu.append((tasks, [page]))
        return True

    def _release_state(self, s: Sequence) -> None:
        if s.state_slot >= 0:
            self.kv.state.release(s.state_slot)
            s.state_slot = -1
        if s.state_item >= 0:
            self.host_state.release(s.state_item)
            s.state_item = -1

    def _complete(self, s: Sequence, reason: str) -> None:
        s.finish_reason = reason
        if not str(reason).startswith("error"):
            self.chunk_sizer.report_completion(s.num_decoded)
        self._release_state(s)
        split = self.model.attn_request_parallel and self.model.layout.tp_size > 1    # decoded KV lives on the owner only
        if self.prefix is not None and s.gpu_pages and s.num_cached_tokens >= self.buf.page_size \
                and not str(reason).startswith("error") and not split:
            # trajectory commit: the full pages of prompt + generated tokens stay in the prefix cache, so a later turn
            # whose prompt extends this one (an agent session) restores them instead of recomputing
            # (batchgen/prefix_reuse/trajectory_commit.py: a finished turn commits its KV up to a page boundary)
            if self.prefix.commit(s.all_ids[: s.num_cached_tokens], s.gpu_pages):
                self.stats.trajectory_commits += 1
            sid = getattr(s, "session_id", None)
            full = s.num_cached_tokens // self.buf.page_size
            if sid and self.trajectories is not None and full >= 1:
                self.kv.alloc.share(s.gpu_pages[:full])                     # the frontier's own references
                self.trajectories.advance(sid, s.all_ids[: s.num_cached_tokens], s.gpu_pages[:full])
                self._session_lru.pop(sid, None)
                self._session_lru[sid] = None
                self.stats.trajectory_frontiers += 1
        if s.gpu_pages:
            self.kv.alloc.free(s.gpu_pages)
            s.gpu_pages = []
        if s.host_pages and self.host_kv is not None:
            self.host_kv.alloc.free(s.host_pages)
            s.host_pages = []
        s.transition(S.COMPLETED)
        if self.on_complete is not None:
            self.on_complete(s)

    # ------------------------------------------------------------------ prefill
    def _prefill_wave(self) -> int:
        """Admit and prefill one wave.  Returns the number of sequences prefilled."""
        cands = self._by_status(S.QUEUEING, S.EVICTED)
        if not cands:
            return 0
        reclaimable = self.prefix.reclaimable_pages() if self.prefix else 0
        segs, ledger = None, None
        if self.prefix is not None:
            # marginal page charges: a page-sized prefix block is paid for by the first prompt that needs it; prompts
            # that share it (in this wave, or through the prefix cache) pay for their private tail only
            segs, ledger, held = {}, sched.SharedPrefixLedger(), set()
            for s in cands:
                keys = self._prefix_keys(s)
                segs[s.global_idx] = [(k, 1) for k in keys]
                for k in keys:
                    page = self.prefix.page_of(k)
                    if page is None:
                        break
                    if page not in held:
                        held.add(page)
                        ledger.charge(0, [(k, 1)])
                        if self.kv.alloc.refcount(page) == 1:
                            reclaimable -= 1               # a hit stays where it is: not part of the budget
        sel = sched.select_prefill_batch(cands, self._free_pages(), self.buf,
                                         reserve_decode_tokens=self.buf.page_size,
                                         prefix_segments=segs, ledger=ledger,
                                         reclaimable_pages=max(reclaimable, 0))
        live = len(self._by_status(S.PREFILLED, S.IN_DECODE, S.ON_HOLD))
        self.guard.observe(len(sel.admitted), live, (len(cands), self._free_pages()))
        admitted = list(sel.admitted)
        if self.kv.state is not None:                 # sequence-slot cap of the recurrent-state pool
            admitted = admitted[: self.kv.state.num_free]
        if not admitted:
            return 0
        t0 = time.perf_counter()
        wave = [self.seqs[i] for i in admitted]
        for s in wave:
            s.transition(S.IN_PREFILL)
        if self.prefix is not None:
            self._prefill_wave_shared(wave)
        else:
            new_lens: List[int] = []
            for s in wave:
                n_total = len(self._prefill_ids(s))
                need = pages_for(n_total + 1, self.buf.page_size)
                s.gpu_pages = self._alloc_pages(need)
                if self.kv.state is not None and s.state_slot < 0:
                    s.state_slot = self.kv.state.acquire()
                s.cached_prefix_tokens = 0
                s.num_cached_tokens = 0
                new_lens.append(n_total)
            # pack into token-capped micro-batches and run them
            for mb in sched.prepack_ffd(new_lens, self.ecfg.max_prefill_tokens):
                self._run_prefill_microbatch([wave[i] for i in mb.seq_indices])
        for s in wave:
            if self.prefix is not None:
                self.prefix.commit(self._prefill_ids(s), s.gpu_pages)
            s.reentry_decoded_baseline = 0
            s.transition(S.PREFILLED)
            fin = s.is_finished(self.cfg.eos_token_id)
            if fin:
                self._complete(s, fin)
        self._sync()
        self.stats.prefill_seconds += time.perf_counter() - t0
        self.stats.prefill_waves += 1
        return len(wave)

    def _promote_from_host(self, ids: Seq[int], pages: List[int]) -> List[int]:
        """Second level of the prefix cache: pages that continue the device hit ``pages`` and were demoted to the
        host tier come back into device pages (asynchronous load, ordered before the prefill on the device) and
        re-enter the device cache.  Returns the extended page list."""
        from .prefix_cache import build_prefix_hash_chain
        ps = self.buf.page_size
        keys = build_prefix_hash_chain(ids[: max(len(ids) - 1, 0)], ps)
        rest = keys[len(pages):]
        if not rest:
            return pages
        host_pages = self.host_tier.lookup(rest)
        if not host_pages:
            return pages
        n = len(host_pages)
        if n > self._free_pages():
            self._reclaim(n - self._free_pages())
        n = min(n, self._free_pages())
        if n == 0:
            self.host_tier.alloc.free(host_pages)
            return pages
        new = self._take_pages(n)
        cur = torch.cuda.current_stream().cuda_stream
        tasks = self.host_tier.load(host_pages[:n], new, after_stream=cur)
        self.host_tier.stream_wait(tasks, cur)
        self._deferred_host.append((tasks, host_pages))           # the caller's references from the lookup
        out = pages + new
        self.prefix.commit(ids[: len(out) * ps], out)               # the device cache takes its own reference
        self.kv.alloc.free(new)
        self.host_tier.promoted_pages += n
        self.stats.prefix_promoted_pages += n
        return out

    def _prefix_keys(self, s: Sequence) -> List[bytes]:
        """Chain keys of the full pages of the tokens a prefill of ``s`` would compute (all but the last token, which
        is always computed); cached on the sequence until its token count changes."""
        from .prefix_cache import build_prefix_hash_chain
        ids = self._prefill_ids(s)
        cached = getattr(s, "_prefix_key_cache", None)
        if cached is None or cached[0] != len(ids):
            cached = (len(ids), build_prefix_hash_chain(ids[: max(len(ids) - 1, 0)], self.buf.page_size))
            s._prefix_key_cache = cached
        return cached[1]

    @staticmethod
    def _prefill_ids(s: Sequence) -> List[int]:
        """Tokens a prefill recomputes: the prompt, plus the tokens decoded before an eviction."""
        return s.all_ids if s.reentry_decoded_baseline else s.prompt_ids

    def _alloc_pages(self, n: int) -> List[int]:
        if n > self._free_pages():
            self._reclaim(n - self._free_pages())
        return self._take_pages(n)

    def _prefill_wave_shared(self, wave: List[Sequence]) -> None:
        """Prefill a wave so that every prefix shared inside it is computed once (in-wave prefix pool), on top of
        the page-level prefix cache that carries prefixes across waves.

        ``wave_plan.plan_wave_prefix_sharing`` cuts the prompts into page-sized blocks, finds the segments that two
        or more prompts pass through and orders the work so that a segment is resident before anything reads it.
        A segment is computed from one member's tokens into pages of its own; every member then holds a reference
        to those pages at the head of its block table and computes only its private tail.  A prompt whose longest
        cached prefix (from an earlier wave or turn) is at least as long as its in-wave chain uses the cached pages
        instead (the planner's *materialized* prefix).  Reference parity: batchgen/prefix_reuse/wave_runtime.py:30-427
        (pool wave: allocate, attach members, commit), executor.py:1-10 (chunk -> prepacked forward with pooled
        ancestors as computed prefix)."""
        ps = self.buf.page_size
        ids_of = [self._prefill_ids(s) for s in wave]
        cached: Dict[int, List[int]] = {}
        hits = []
        for i, ids in enumerate(ids_of):
            pages, _ = self.prefix.lookup(ids)
            if self.host_tier is not None:
                pages = self._promote_from_host(ids, pages)
            if pages:
                cached[i] = pages
                hits.append(wave_plan.MaterializedPrefix(i, len(pages) * ps))
        plan = wave_plan.plan_wave_prefix_sharing(ids_of, ps, threshold=2, chunk_tokens=self.ecfg.max_prefill_tokens,
                                                  materialized=hits)
        seg_pages: Dict[int, List[int]] = {}
        for chunk in plan.chunks:
            rows: List[_PrefillRow] = []
            for idx in chunk:
                it = plan.items[idx]
                chain: List[int] = []
                for sid in it.prefix_segments:
                    chain += seg_pages[sid]
                if it.kind == "materialize":
                    seg = plan.segments[it.ref]
                    pages = cached[seg.members[0]][: seg.tokens // ps]
                    self.prefix.attach(pages)                     # the pool's own reference, dropped below
                    seg_pages[it.ref] = pages
                elif it.kind == "segment":
                    seg = plan.segments[it.ref]
                    own = self._alloc_pages(seg.tokens // ps)
                    seg_pages[it.ref] = own
                    rows.append(_PrefillRow(ids_of[seg.members[0]][it.token_start:it.token_end], it.token_start,
                                            chain + own))
                    self.stats.shared_prefix_tokens += (len(seg.members) - 1) * seg.tokens
                else:
                    s = wave[it.ref]
                    n_total = len(ids_of[it.ref])
                    own = self._alloc_pages(pages_for(n_total + 1, ps) - it.token_start // ps)
                    self.kv.alloc.share(chain)                    # this member's references to the shared pages
                    s.gpu_pages = chain + own
                    s.cached_prefix_tokens = it.token_start
                    s.num_cached_tokens = it.token_start
                    rows.append(_PrefillRow(ids_of[it.ref][it.token_start:], it.token_start, s.gpu_pages, s))
            if rows:
                self._run_prefill_rows(rows)
        for pages in seg_pages.values():
            self.kv.alloc.free(pages)

    def _run_prefill_microbatch(self, group: List[Sequence]) -> None:
        rows = []
        for s in group:
            full = self._prefill_ids(s)
            rows.append(_PrefillRow(full[s.num_cached_tokens:], s.num_cached_tokens, s.gpu_pages, s))
        self._run_prefill_rows(rows)

    def _run_prefill_rows(self, rows: List[_PrefillRow]) -> None:
        """Prefill ``rows``; rows that belong to a sequence get their first token sampled.  A row longer than
        ``max_prefill_tokens`` is computed in pieces over consecutive forwards (chunked prefill: every piece attends
        over the KV its predecessors wrote; only the last piece produces a token), so activation memory is bounded
        by the cap whatever the prompt length (batchgen/prefill.py: chunked long-context prefill)."""
        cap = max(int(self.ecfg.max_prefill_tokens), 1)
        if not any(len(r.tokens) > cap for r in rows):
            return self._run_prefill_forward(rows)
        pending = [(r, 0) for r in rows]
        while pending:
            batch: List[_PrefillRow] = []
            later = []
            used = 0
            for r, off in pending:
                room = cap - used
                if room <= 0:
                    later.append((r, off))
                    continue
                n = min(len(r.tokens) - off, room)
                last = off + n == len(r.tokens)
                batch.append(_PrefillRow(r.tokens[off:off + n], r.start + off, r.pages, r.seq if last else None,
                                         state_slot=r.state_slot))
                used += n
                if not last:
                    later.append((r, off + n))
            self._run_prefill_forward(batch)
            self.stats.prefill_chunks += 1
            pending = later

    def _run_prefill_forward(self, rows: List[_PrefillRow]) -> None:
        """One packed prefill forward over ``rows``."""
        ps = self.buf.page_size
        ids: List[int] = []
        pos: List[int] = []
        slots: List[int] = []
        cu = [0]
        ctx_lens: List[int] = []
        for r in rows:
            a, b = r.start, r.start + len(r.tokens)
            ids += r.tokens
            pos += list(range(a, b))
            slots += slots_for_range(r.pages, a, b, ps)
            cu.append(cu[-1] + (b - a))
            ctx_lens.append(a)
        dev = self.device
        T = len(ids)
        W = self.sp_world
        pad = (-T) % W                                # fused path: whole rows-per-rank blocks; padding rows write no KV
        if pad:
            ids += [0] * pad
            pos += [0] * pad
            slots += [-1] * pad
        group = [r.seq for r in rows if r.seq is not None]
        logit_rows = [cu[i + 1] - 1 for i, r in enumerate(rows) if r.seq is not None]
        has_state = self.kv.state is not None
        meta = AttnMeta(
            mode="prefill",
            positions=torch.tensor(pos, dtype=torch.int32, device=dev),
            slot_mapping=torch.tensor(slots, dtype=torch.int64, device=dev),
            block_table=build_block_table([r.pages for r in rows], dev),
            cu_seqlens=cu, ctx_lens=ctx_lens,
            state_slots=(torch.tensor([r.state_slot for r in rows], dtype=torch.int32, device=dev)
                         if has_state else None),
            state_has_initial=(torch.tensor([int(c > 0) for c in ctx_lens], dtype=torch.int32, device=dev)
                               if has_state else None),
            logit_rows=torch.tensor(logit_rows, dtype=torch.int64, device=dev),
            num_valid=torch.tensor([T], dtype=torch.int32, device=dev) if W > 1 else None)
        ids_t = torch.tensor(ids, dtype=torch.int32, device=dev)
        self.stats.prefill_tokens += T
        self.step_ring.record("prefill", len(rows), T)
        if W > 1:
            logits = self.model.forward_sp(ids_t, meta, self.kv)      # wanted rows that this rank owns
            toks = self._sample_sharded(logits, group, logit_rows, T + pad) if group else []
        else:
            logits = self.model.forward(ids_t, meta, self.kv)
            toks = self._sample(logits, group).tolist() if group else []
        for s, t in zip(group, toks):
            self.stats.prefill_cached_tokens += s.cached_prefix_tokens
            s.num_cached_tokens = len(self._prefill_ids(s))
            s.output_ids.append(int(t))

    # ------------------------------------------------------------------ sampling
    @staticmethod
    def _greedy_row(s: Optional[Sequence]) -> bool:
        return s is None or s.params.temperature <= 0

    def _sample(self, logits: torch.Tensor, rows: List[Optional[Sequence]], resident: bool = False,
                uniform: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Tokens for ``logits`` rows; ``rows[i]`` owns row i (``None`` = padding row, sampled greedily and dropped
        by the caller).  ``resident``: the per-row parameters come from the device-resident cache, which is
        re-uploaded only when the ordered row set changes (decode steps)."""
        if all(self._greedy_row(s) for s in rows):
            return sampling_ops.greedy(logits, out)
        dev = logits.device
        if resident:
            key = tuple(s.global_idx if s is not None else -1 for s in rows)
            if key != self._samp_key:                  # rebind (never mutate) on change: the cache keys on identity
                self._samp_key, self._samp_rows = key, list(rows)
                self._samp_epoch += 1
            prm = [dict(temperature=0.0, top_p=1.0, top_k=0) if s is None else s.params for s in self._samp_rows]
            v = self._residency.view(self._samp_rows, prm, self._samp_epoch, 0)
            temp, tk, tp = v.temperature, v.top_k, v.top_p
        else:
            temp = torch.tensor([0.0 if s is None else s.params.temperature for s in rows], dtype=torch.float32,
                                device=dev)
            tk = torch.tensor([0 if s is None else s.params.top_k for s in rows], dtype=torch.int32, device=dev)
            tp = torch.tensor([1.0 if s is None else s.params.top_p for s in rows], dtype=torch.float32, device=dev)
        return sampling_ops.sample(logits, temp, tk, tp, uniform=uniform, out=out, generator=self._gen)

    def _sample_sharded(self, logits: torch.Tensor, rows: List[Optional[Sequence]], row_index: List[int],
                        padded_rows: int, resident: bool = False) -> List[int]:
        """Fused sequence-parallel path.  ``logits`` holds, in order, the wanted rows that this rank owns: wanted
        row i is row ``row_index[i]`` (ascending) of the padded step and belongs to rank ``row_index[i] //
        (padded_rows / world)``.  Every rank samples its own rows, then one all-gather gives every rank every
        token.  Random draws use one uniform number per wanted row taken from the generator that all ranks seed
        alike, so the result does not depend on which rank owns a row."""
        import torch.distributed as dist
        comm = self.model.comm
        W, r = self.sp_world, comm.rank
        Tl = padded_rows // W
        owners = [j // Tl for j in row_index]
        counts = [0] * W
        for o in owners:
            counts[o] += 1
        maxc = max(counts) if counts else 0
        dev = self.device
        if maxc == 0:
            return []
        tok_local = torch.zeros(maxc, dtype=torch.int32, device=dev)
        mine = [i for i, o in enumerate(owners) if o == r]
        uniform = None
        if not all(self._greedy_row(s) for s in rows):
            u_all = torch.rand(len(rows), device=dev, generator=self._gen)      # the same numbers on every rank
            uniform = u_all[torch.tensor(mine, dtype=torch.long, device=dev)] if mine else None
        if mine:
            self._sample(logits, [rows[i] for i in mine], resident=resident, uniform=uniform,
                         out=tok_local[: len(mine)])
        gathered = torch.empty(W * maxc, dtype=torch.int32, device=dev)
        dist.all_gather_into_tensor(gathered, tok_local, group=getattr(comm, "group", None))
        g = gathered.view(W, maxc).tolist()
        cursor = [0] * W
        toks = []
        for o in owners:
            toks.append(g[o][cursor[o]])
            cursor[o] += 1
        return toks

    # ------------------------------------------------------------------ decode
    def _enter_decode(self, s: Sequence) -> bool:
        """Make sure the row's KV and growth buffer are on the GPU; returns False if it does not fit."""
        want = gpu_pages_first_load(s.context_len, self.buf, self.kv_token_budget)
        if s.state_item >= 0 and self.kv.state.num_free == 0:
            return False                              # no slot for the parked state yet
        if s.host_pages and not s.gpu_pages:          # parked in the host tier: load back
            need = max(want, len(s.host_pages))
            if need > self._free_pages():
                self._reclaim(need - self._free_pages())
            if need > self._free_pages():
                return False
            s.gpu_pages = self._take_pages(need)
            if self.host_tier is not None:
                # asynchronous load: the compute stream waits on the device, the host goes on; the host pages are
                # released when the copy is done
                cur = torch.cuda.current_stream().cuda_stream   # after the kernels that may still read these pages
                tasks = self.host_tier.load(s.host_pages, s.gpu_pages[: len(s.host_pages)], after_stream=cur)
                self.host_tier.stream_wait(tasks, cur)
                self._deferred_host.append((tasks, s.host_pages))
                s.host_pages = []
                self.stats.loads += 1
            else:
                self.kv.copy_pages_from(self.host_kv, s.host_pages, s.gpu_pages[: len(s.host_pages)], self.copy_stream)
            if s.state_item >= 0:
                s.state_slot = self.kv.state.acquire()
                self.host_state.load(self.kv.state, s.state_item, s.state_slot, self.copy_stream)
                self.host_state.release(s.state_item)
                s.state_item = -1
            if s.host_pages:
                if self.copy_stream is not None:
                    torch.cuda.current_stream().wait_stream(self.copy_stream)
                self.host_kv.alloc.free(s.host_pages)
                s.host_pages = []
                self.stats.loads += 1
        extra = want - len(s.gpu_pages)
        if extra > 0:
            if extra > self._free_pages():
                self._reclaim(extra - self._free_pages())
            if extra > self._free_pages():
                return False
            s.gpu_pages += self._take_pages(extra)
        s.had_initial_gpu_reservation = True
        s.transition(S.IN_DECODE)
        return True

    def _hold(self, s: Sequence) -> None:
        """Take a row out of the decode batch; move its KV to the host tier when there is one."""
        used = pages_for(s.num_cached_tokens, self.buf.page_size)
        if self.host_tier is not None and self._deferred_host and self.host_tier.alloc.num_free < used:
            self._drain_deferred(block=True)           # host pages of finished loads
        if self.host_kv is not None and self.host_kv.alloc.num_free < used:
            self._make_host_room(s, used)
        if self.host_tier is not None and self.host_tier.alloc.num_free >= used:
            # asynchronous offload after the kernels that wrote the KV; the device pages return to the pool when
            # the copy is done (no host synchronisation here)
            s.host_pages = self.host_tier.alloc.alloc(used)
            tasks = self.host_tier.offload(s.gpu_pages[:used], s.host_pages,
                                           after_stream=torch.cuda.current_stream().cuda_stream)
            self._deferred_gpu.append((tasks, s.gpu_pages))
            s.gpu_pages = []
            self.stats.offloaded_pages += used
            s.transition(S.ON_HOLD)
            self.stats.holds += 1
        elif self.host_tier is None and self.host_kv is not None and self.host_kv.alloc.num_free >= used:
            s.host_pages = self.host_kv.alloc.alloc(used)
            self.host_kv.copy_pages_from(self.kv, s.gpu_pages[:used], s.host_pages, self.copy_stream)
            if self.host_state is not None and s.state_slot >= 0 and self.host_state.num_free:
                if self.copy_stream is not None:
                    self.copy_stream.wait_stream(torch.cuda.current_stream())
                s.state_item = self.host_state.offload(self.kv.state, s.state_slot, self.copy_stream)
            if self.copy_stream is not None:
                self.copy_stream.synchronize()
            if s.state_item >= 0:                      # the slot goes to whoever is scheduled next
                self.kv.state.release(s.state_slot)
                s.state_slot = -1
            self.kv.alloc.free(s.gpu_pages)
            s.gpu_pages = []
            self.stats.offloaded_pages += used
            s.transition(S.ON_HOLD)
            self.stats.holds += 1
        else:
            self._evict(s)

    def _make_host_room(self, s: Sequence, need: int) -> None:
        """The host tier cannot take ``need`` more pages for row ``s``: parked rows give theirs up, cheapest to
        recompute first (they fall back to EVICTED and are re-prefilled later), only as many as the debt requires
        (batchgen/continuous_batching.py:578-700: eviction is strictly growth driven)."""
        from .continuous_batching import EvictionStrategy, plan_host_kv_growth_evictions
        held = [q for q in self.seqs.values() if q.status == S.ON_HOLD and q.host_pages and q is not s]
        if not held:
            return
        total = self.host_kv.num_pages
        plan = plan_host_kv_growth_evictions(
            active_uuids=[str(q.global_idx) for q in held] + [str(s.global_idx)], completed_uuids=[],
            host_growth_uuids=[str(s.global_idx)], host_growth_pages=[need],
            eviction_candidates=[(str(q.global_idx), dict(host_owned_pages=len(q.host_pages),
                                                          decoded_length=q.num_decoded, global_idx=q.global_idx))
                                 for q in held],
            free_pages=self.host_kv.alloc.num_free, total_pages=total, completed_pages=0,
            strategy=EvictionStrategy.SHORTEST_FIRST)
        if not plan.growth_feasible_after_eviction:
            return                                     # evicting everybody would still not fit: ``s`` is evicted instead
        for uid in plan.evicted_uuids:
            self._evict(self.seqs[int(uid)])
            self.stats.growth_evictions += 1

    def _evict(self, s: Sequence) -> None:
        if s.gpu_pages:
            self.kv.alloc.free(s.gpu_pages)
        if s.host_pages and self.host_kv is not None:
            self.host_kv.alloc.free(s.host_pages)
        self._release_state(s)
        s.evict()
        s.output_ids = list(s.output_ids)     # decoded tokens are kept and replayed through prefill
        self.stats.evictions += 1

    def _owner_layout(self, rows: List[Sequence]) -> List[Optional[Sequence]]:
        """Request-split decode attention: arrange the step's rows in one block per TP rank (a row always in
        the block of its owner, the rank whose KV copy its decode steps extend) and pad every block to the same
        length with empty rows (``None``).  A new row goes to the rank that owns the fewest live rows; every
        rank runs this same code on the same inputs, so all agree without talking."""
        W = self.model.layout.tp_size
        load = [0] * W
        for s in self.seqs.values():
            if s.decode_owner >= 0 and s.status in (S.PREFILLED, S.IN_DECODE, S.ON_HOLD):
                load[s.decode_owner] += 1
        blocks: List[List[Sequence]] = [[] for _ in range(W)]
        for s in rows:
            if s.decode_owner < 0:
                s.decode_owner = min(range(W), key=lambda r: (load[r], r))
                load[s.decode_owner] += 1
            blocks[s.decode_owner].append(s)
        per = max(len(b) for b in blocks)
        if self.graph_runner is not None:                # the whole step must be one of the captured sizes
            per = -(-self.graph_runner.bucketing.bucket_for(W * per) // W)
        layout: List[Optional[Sequence]] = []
        for b in blocks:
            layout += b + [None] * (per - len(b))
        return layout

    def _step_layout(self, rows: List[Sequence]):
        """(layout, positions, KV slots, lengths) of one decode step over ``rows``; ``None`` layout entries are
        padding rows."""
        ps = self.buf.page_size
        W = self.sp_world
        split = self.model.attn_request_parallel and self.model.layout.tp_size > 1
        layout: List[Optional[Sequence]] = self._owner_layout(rows) if split else list(rows)
        if W > 1 and self.graph_runner is None and len(layout) % W:
            layout += [None] * ((-len(layout)) % W)      # fused path: whole rows-per-rank blocks
        pos = [s.num_cached_tokens if s is not None else 0 for s in layout]
        slots = [s.gpu_pages[p // ps] * ps + p % ps if s is not None else -1 for s, p in zip(layout, pos)]
        lens = [p + 1 if s is not None else 0 for s, p in zip(layout, pos)]
        return layout, pos, slots, lens

    def _decode_step(self, rows: List[Sequence]) -> None:
        """One synchronous decode step (the path without captured graphs)."""
        dev = self.device
        W = self.sp_world
        split = self.model.attn_request_parallel and self.model.layout.tp_size > 1
        layout, pos, slots, lens = self._step_layout(rows)
        ids = [s.all_ids[s.num_cached_tokens] if s is not None else 0 for s in layout]
        if self.graph_runner is not None:
            logits, bucket = self.graph_runner.decode(self, layout, ids, pos, slots, lens)
            if W > 1:
                layout = layout + [None] * (bucket - len(layout))    # the captured step covers the whole bucket
        else:
            n_real = sum(1 for s in layout if s is not None)
            meta = AttnMeta(
                mode="decode",
                positions=torch.tensor(pos, dtype=torch.int32, device=dev),
                slot_mapping=torch.tensor(slots, dtype=torch.int64, device=dev),
                block_table=build_block_table([s.gpu_pages if s is not None else [] for s in layout], dev),
                seqlens=torch.tensor(lens, dtype=torch.int32, device=dev),
                state_slots=(torch.tensor([s.state_slot if s is not None else -1 for s in layout], dtype=torch.int32,
                                          device=dev) if self.kv.state is not None else None))
            ids_t = torch.tensor(ids, dtype=torch.int32, device=dev)
            if W > 1:
                if not split and n_real != len(layout):
                    # padding rows sit at the end: the router skips them (request-split layouts pad inside the
                    # blocks instead; there the empty rows are routed like any row and dropped afterwards)
                    meta.num_valid = torch.tensor([n_real], dtype=torch.int32, device=dev)
                logits = self.model.forward_sp(ids_t, meta, self.kv)
            else:
                logits = self.model.forward(ids_t, meta, self.kv)
        if W > 1:
            toks = self._sample_sharded(logits, layout, list(range(len(layout))), len(layout), resident=True)
        else:
            toks = self._sample(logits, layout, resident=True).tolist()
        n = 0
        for s, t in zip(layout, toks):
            if s is None:
                continue
            s.num_cached_tokens += 1
            s.output_ids.append(int(t))
            n += 1
        self.stats.decode_tokens += n
        self.stats.decode_steps += 1

    # -------- deferred read-back: the host sees a step's tokens while the next step already runs
    def _launch_decode(self, rows: List[Sequence], feed_key) -> dict:
        """Enqueue one captured decode step and the device-side sampling without waiting for the result.  When the
        step's layout equals ``feed_key`` (the layout of the step launched just before), its input tokens are the
        ones that step sampled, taken on the device; otherwise they come from the host.  The reference keeps the same
        one-step lag (batchgen/worker/deferred_readback.py:57)."""
        runner = self.graph_runner
        W = self.sp_world
        layout, pos, slots, lens = self._step_layout(rows)
        key = tuple(s.global_idx if s is not None else -1 for s in layout)
        ids = None if key == feed_key else [s.all_ids[s.num_cached_tokens] if s is not None else 0 for s in layout]
        logits, bucket = runner.decode(self, layout, ids, pos, slots, lens)
        n = len(layout)
        if W > 1:
            import torch.distributed as dist
            comm = self.model.comm
            full = layout + [None] * (bucket - n)
            Tl = bucket // W
            mine = full[comm.rank * Tl:(comm.rank + 1) * Tl]
            uniform = None
            if not all(self._greedy_row(s) for s in full):
                u_all = torch.rand(bucket, device=self.device, generator=self._gen)   # the same numbers on every rank
                uniform = u_all[comm.rank * Tl:(comm.rank + 1) * Tl]
            tl = runner._tok_local[:Tl]
            self._sample(logits[:Tl], mine, resident=True, uniform=uniform, out=tl)
            dist.all_gather_into_tensor(runner.tokens[:bucket], tl, group=getattr(comm, "group", None))
        else:
            self._sample(logits, layout, resident=True, out=runner.tokens[:n])
        handle = runner.start_readback(n)
        for s in layout:
            if s is not None:
                s.num_cached_tokens += 1
                s.inflight_tokens += 1
        self.stats.decode_steps += 1
        return dict(layout=layout, key=key, handle=handle, rows=[s.global_idx for s in rows])

    def _retire_decode(self, pending: dict) -> None:
        """Bring a launched step's tokens to the host and append them to their rows.  A row that had already ended
        when the step was launched (its end-of-sequence token became visible one step late) drops the extra token."""
        toks = self.graph_runner.read(pending["handle"]).tolist()
        eos = self.cfg.eos_token_id
        n = 0
        for s, t in zip(pending["layout"], toks):
            if s is None:
                continue
            s.inflight_tokens -= 1
            if s.inflight_tokens == 0 and s.is_finished(eos):
                continue
            s.output_ids.append(int(t))
            n += 1
        self.stats.decode_tokens += n

    def _decode_interval(self, max_steps: Optional[int] = None) -> int:
        """Admit rows, decode up to one decision interval, then apply the boundary decisions.
        Returns the number of decode steps executed."""
        free = {0: self._free_pages() + (self.prefix.reclaimable_pages() if self.prefix else 0)}
        in_dec = self._by_status(S.IN_DECODE)
        admit = sched.select_decode_batch(self.seqs.values(), free, {0: len(in_dec)}, self.ecfg.max_decode_batch,
                                          self.buf, self.kv_token_budget, total_pages_per_bucket=self.kv.num_pages,
                                          resident={s.global_idx for s in self.seqs.values() if s.gpu_pages})
        for gi in admit:
            self._enter_decode(self.seqs[gi])
        rows = sorted(self._by_status(S.IN_DECODE), key=lambda s: s.global_idx)
        if not rows:
            return 0
        t0 = time.perf_counter()
        steps = 0
        eos = self.cfg.eos_token_id
        limit = min(self.buf.decision_interval, max_steps or self.buf.decision_interval)
        deferred = self.graph_runner is not None and self.ecfg.deferred_readback
        pending: Optional[dict] = None

        def launchable(s: Sequence) -> bool:
            return (not s.is_finished(eos)
                    and s.num_decoded + s.inflight_tokens < s.params.max_new_tokens)

        for _ in range(limit):
            live = [s for s in rows if launchable(s)]
            if not live:
                break
            # a row about to cross into a page it does not own ends the interval early
            if any(pages_for(s.num_cached_tokens + 1, self.buf.page_size) > len(s.gpu_pages) for s in live):
                break
            if not deferred:
                self._decode_step(live)
            else:
                if pending is not None and pending["rows"] != [s.global_idx for s in live]:
                    # the batch changes: its input tokens come from the host, so the step in flight lands first
                    self._retire_decode(pending)
                    pending = None
                    live = [s for s in live if launchable(s)]
                    if not live:
                        break
                nxt = self._launch_decode(live, pending["key"] if pending is not None else None)
                if pending is not None:
                    self._retire_decode(pending)
                pending = nxt
            steps += 1
            self.step_ring.record("decode", len(live), len(live))
            if self.step_hook is not None:
                self.step_hook("decode")
        if pending is not None:
            self._retire_decode(pending)
        self._sync()
        self.stats.decode_seconds += time.perf_counter() - t0
        self._apply_boundary()
        return steps

    def _apply_boundary(self) -> None:
        free_host = self.host_kv.alloc.num_free if self.host_kv is not None else 0
        d = sched.compute_boundary_decisions(
            list(self.seqs.values()), self.cfg.eos_token_id, {0: self._free_pages()}, free_host, self.buf,
            self.kv_token_budget, self.ecfg.max_decode_batch, self.chunk_sizer.get_chunk_size(), host_tier=False,
            reclaimable_host_pages=0)
        if d.scheduler_error:
            raise RuntimeError(d.scheduler_error)
        for gi in d.completed:
            s = self.seqs[gi]
            self._complete(s, s.is_finished(self.cfg.eos_token_id))
        for gi in d.on_hold:
            self._hold(self.seqs[gi])
        for gi, extra in d.extend.items():
            s = self.seqs[gi]
            if s.status != S.IN_DECODE:
                continue
            if extra > self._free_pages():
                self._reclaim(extra - self._free_pages())
            if extra > self._free_pages():
                self._hold(s)
                continue
            s.gpu_pages += self._take_pages(extra)
        for gi in d.load:
            s = self.seqs[gi]
            if s.status in (S.PREFILLED, S.ON_HOLD):
                self._enter_decode(s)

    # ------------------------------------------------------------------ main loop
    def has_work(self) -> bool:
        return any(s.status != S.COMPLETED for s in self.seqs.values())

    def step(self) -> None:
        """One scheduling action: a prefill wave when nothing is decodable or free pages allow more
        admissions, otherwise one decode interval."""
        waiting = self._by_status(S.QUEUEING, S.EVICTED)
        decodable = self._by_status(S.PREFILLED, S.IN_DECODE, S.ON_HOLD)
        did = 0
        if waiting and (not decodable or self._prefill_headroom(waiting)):
            did = self._prefill_wave()
        if self._by_status(S.PREFILLED, S.IN_DECODE, S.ON_HOLD):
            steps = self._decode_interval()
            if steps == 0 and did == 0:
                self._break_deadlock()
        elif did == 0 and waiting:
            self._break_deadlock()

    def _prefill_headroom(self, waiting: List[Sequence]) -> bool:
        """Is it worth leaving decode for another wave?  Yes when the decode batch has free rows and
        the smallest waiting prompt fits the free pages (the watermark rule of the reference,
        batchgen/worker/kv_manager.py:632-670, applied to the device pool)."""
        if len(self._by_status(S.IN_DECODE)) >= self.ecfg.max_decode_batch:
            return False
        free_frac = self._free_pages() / max(1, self.kv.num_pages)
        if not sched.watermark_trigger([free_frac], 100 - self.ecfg.host_kv_watermark, True, False):
            return False
        smallest = min(s.context_len for s in waiting)
        return pages_for(smallest + self.buf.page_size, self.buf.page_size) <= self._free_pages()

    def _break_deadlock(self) -> None:
        """Nothing could run: free space by evicting the parked row with the least decoded work."""
        parked = self._by_status(S.ON_HOLD, S.PREFILLED)
        if parked:
            v = min(parked, key=lambda s: (s.num_decoded, s.global_idx))
            self._evict(v)
            return
        stuck = self._by_status(S.IN_DECODE)
        if stuck:
            # rows that can neither grow (context budget exhausted) nor be parked: finish them
            for s in stuck:
                if pages_for(s.num_cached_tokens + 1, self.buf.page_size) > len(s.gpu_pages):
                    self._complete(s, "length")
            return
        waiting = self._by_status(S.QUEUEING, S.EVICTED)
        if waiting:
            s = min(waiting, key=lambda s: s.context_len)
            if pages_for(s.context_len + 1, self.buf.page_size) > self.kv.num_pages:
                s.status = S.COMPLETED
                s.finish_reason = "error: prompt does not fit the KV pool"
                if self.on_complete:
                    self.on_complete(s)

    def run_to_completion(self, max_iterations: int = 1_000_000) -> List[Sequence]:
        it = 0
        while self.has_work():
            self.step()
            it += 1
            if it > max_iterations:
                raise RuntimeError("engine did not converge")
        return sorted(self.seqs.values(), key=lambda s: s.global_idx)

    def generate(self, prompts: Seq[Seq[int]], params=None) -> List[List[int]]:
        """Token ids generated for every prompt; ``params`` is one ``SamplingParams`` for all or one per prompt."""
        per = list(params) if isinstance(params, (list, tuple)) else [params] * len(prompts)
        seqs = [self.add_request(p, q) for p, q in zip(prompts, per)]
        self.run_to_completion()
        return [s.output_ids for s in seqs]
