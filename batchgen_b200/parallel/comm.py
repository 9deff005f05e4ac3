"""Communication layer seen by the model: ``tp_reduce``, ``tp_gather_vocab`` and ``moe``.

Two implementations share the interface:

* ``NcclComm`` — the *baseline*: plain NCCL collectives around local kernels, reproducing the
  reference's decode dataflow ``all_gather(tokens) -> route on global tokens -> local experts ->
  reduce_scatter`` (batchgen/models/glm/glm5/model.py:2391-2508,
  batchgen/models/deepseek/deepseekv3/modeling_deepseek_v3.py:3046-3200) and all_reduce after the
  tensor-parallel o_proj (batchgen/models/moonshotai/kimi_linear/Parallel_Strategy_Manager.py:684-808).
* ``FusedComm`` (``parallel/fused.py``) — the product: kernels that move data over NVLink
  themselves (peer stores / multimem) fused with quantisation, GEMM epilogues and the weighted
  combine.

Both work with the ``gloo`` backend on CPU tensors, which is how the multi-rank logic is tested
without GPUs.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ..ops import moe as moe_ops
from ..ops.moe import ExpertWeights


class NcclComm:
    def __init__(self, group=None, rank: Optional[int] = None, world: Optional[int] = None):
        self.group = group
        self.rank = dist.get_rank(group) if rank is None else rank
        self.world = dist.get_world_size(group) if world is None else world
        self.bytes_sent = 0

    # ---- tensor parallel
    def tp_reduce(self, x: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return x
        x = x.contiguous()
        dist.all_reduce(x, group=self.group)
        self.bytes_sent += x.numel() * x.element_size()
        return x

    def tp_gather_vocab(self, logits: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return logits
        parts = [torch.empty_like(logits) for _ in range(self.world)]
        dist.all_gather(parts, logits.contiguous(), group=self.group)
        return torch.cat(parts, dim=-1)

    def all_to_all(self, x: torch.Tensor) -> torch.Tensor:
        """x [world, ...]: slice d goes to rank d; returns [world, ...] with slice s received from rank s."""
        if self.world == 1:
            return x
        x = x.contiguous()
        out = torch.empty_like(x)
        dist.all_to_all_single(out, x, group=self.group)
        self.bytes_sent += x.numel() * x.element_size() * (self.world - 1) // self.world
        return out

    def a2a_rows_to_ranks(self, x: torch.Tensor) -> torch.Tensor:
        """x [world * n, c] (block d of n rows is bound for rank d) -> [n, world, c]: for each of this rank's n rows,
        the c-wide piece every rank holds of it."""
        W = self.world
        n = x.shape[0] // W
        return self.all_to_all(x.view(W, n, -1)).transpose(0, 1).contiguous()

    def a2a_ranks_to_rows(self, x: torch.Tensor) -> torch.Tensor:
        """The inverse exchange: x [n, world, c] (piece d of every row returns to rank d) -> [world * n, c]."""
        n, W, c = x.shape
        return self.all_to_all(x.transpose(0, 1).contiguous()).view(W * n, c)

    def all_gather_rows(self, x: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return x
        out = torch.empty(self.world * x.shape[0], *x.shape[1:], dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous(), group=self.group)
        return out

    def reduce_scatter_rows(self, x: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return x
        out = torch.empty(x.shape[0] // self.world, *x.shape[1:], dtype=x.dtype, device=x.device)
        if x.is_cuda:
            dist.reduce_scatter_tensor(out, x.contiguous(), group=self.group)
        else:  # gloo has no reduce_scatter
            y = x.contiguous().clone()
            dist.all_reduce(y, group=self.group)
            out.copy_(y[self.rank * out.shape[0]:(self.rank + 1) * out.shape[0]])
        return out

    # ---- expert parallel
    def moe(self, hidden: torch.Tensor, topk_idx: torch.Tensor, topk_w: torch.Tensor, ew: ExpertWeights,
            num_experts: int, num_valid=None, replicated: bool = True) -> torch.Tensor:
        """Expert-parallel MoE over NCCL.

        ``replicated`` (tensor-parallel attention): every rank already holds the same rows, so each
        rank runs its local experts over all rows and the partial sums are all-reduced.
        Otherwise (data-parallel attention) rows are all-gathered first and the partial outputs
        reduce-scattered back to their owners."""
        per = num_experts // self.world
        lo, hi = self.rank * per, (self.rank + 1) * per
        if replicated:
            part = moe_ops.experts_forward(hidden, topk_idx, topk_w, ew, lo, hi, num_valid=num_valid)
            return self.tp_reduce(part)
        h = self.all_gather_rows(hidden)
        idx = self.all_gather_rows(topk_idx)
        w = self.all_gather_rows(topk_w)
        part = moe_ops.experts_forward(h, idx, w, ew, lo, hi)
        return self.reduce_scatter_rows(part)


def init_distributed(backend: Optional[str] = None) -> NcclComm:
    """Join the job described by RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT."""
    import os
    if not dist.is_initialized():
        backend = backend or ("nccl" if torch.cuda.is_available() else "gloo")
        if backend == "nccl":
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        dist.init_process_group(backend=backend)
    return NcclComm()
