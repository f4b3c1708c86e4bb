"""Expert-parallel MoE FFN over one node: 256/N experts per rank, one process per GPU.

The reference runs on one GPU and streams experts from SSD; sharding experts across
GPUs is new here.  Per layer and step:

  1. all-gather of the ranks' own rows of x (the dense form of the token dispatch:
     decode batches are a few KB per rank, and with top-8 over <= 8 ranks nearly
     every rank needs every row anyway);
  2. every rank scores the router for all rows (the router is replicated and tiny)
     and runs its LOCAL experts on the rows routed to them, producing one fp32 share
     row per token (zero where it holds none of the token's experts);
  3. all-to-all of the share rows back to the rank that owns each token (the
     combine); the owner adds the shares in rank order, its shared-expert output and
     the residual.

The collectives go through a torch.distributed group (NCCL on GPUs over
NVLink/NVSwitch, gloo in the CPU tests); the arithmetic goes through a backend
object, so the same driver runs on the CUDA library and on the CPU oracle.
"""
from __future__ import annotations

from dataclasses import dataclass

NOT_LOCAL = 0xFFFFFFFF


@dataclass
class ExpertPlacement:
    """Which rank holds which expert.  "contiguous": rank r holds experts
    [r*E/N, (r+1)*E/N).  "strided": expert e lives on rank e mod N, which spreads a
    skewed (Zipf) popularity over the ranks."""
    num_experts: int
    world: int
    mode: str = "contiguous"

    def __post_init__(self):
        if self.num_experts % self.world:
            raise ValueError(f"{self.num_experts} experts do not split over {self.world} ranks")
        if self.mode not in ("contiguous", "strided"):
            raise ValueError(self.mode)
        self.per_rank = self.num_experts // self.world

    def owner(self, e: int) -> int:
        return e // self.per_rank if self.mode == "contiguous" else e % self.world

    def local_index(self, e: int) -> int:
        return e % self.per_rank if self.mode == "contiguous" else e // self.world

    def local_experts(self, rank: int) -> list[int]:
        """Global ids of the rank's blobs, in local-index order."""
        return sorted((e for e in range(self.num_experts) if self.owner(e) == rank), key=self.local_index)

    def expert_map(self, rank: int) -> list[int]:
        return [self.local_index(e) if self.owner(e) == rank else NOT_LOCAL for e in range(self.num_experts)]

    def pairs_per_rank(self, idx) -> list[int]:
        """Load of a routing: number of (token, expert) pairs each rank serves."""
        load = [0] * self.world
        for e in idx:
            load[self.owner(int(e))] += 1
        return load


def ep_layer_step(backend, dist, group, layer: int, x_own, *, world: int):
    """One layer for this rank's rows.  x_own: [B_own, D] fp16 tensor.  Returns y
    [B_own, D] (the block output before the residual add) in the backend's output type."""
    import torch
    b_own = x_own.shape[0]
    x_all = torch.empty((world * b_own, x_own.shape[1]), dtype=x_own.dtype, device=x_own.device)
    dist.all_gather_into_tensor(x_all, x_own.contiguous(), group=group)
    idx, w = backend.router(layer, x_all)
    share = backend.routed_partial(layer, x_all, idx, w)             # [world*B_own, D] fp32
    recv = torch.empty_like(share)
    dist.all_to_all_single(recv, share, group=group)                 # chunk r of my shares -> rank r
    h1 = backend.shared(layer, x_own)
    return backend.finalize(recv, h1, world, b_own)


def ep_stack_step(backend, dist, group, x_own, *, world: int, layers: int):
    """The FFN-only stack of the benchmark: layers chained by the RMS renormalisation."""
    x = x_own
    y = None
    for layer in range(layers):
        y = ep_layer_step(backend, dist, group, layer, x, world=world)
        if layer + 1 < layers:
            x = backend.renorm(y)
    return y


def ep_replicated_stack_step(backend, dist, group, x_own, *, world: int, layers: int):
    """The step structure of the fused expert-parallel decode kernel (up to 8 rows in total), written with
    collectives: ONE all-gather of the rows, then per layer every rank routes ALL rows, computes the shares of the
    pairs whose expert it holds and the shared expert for all rows, the shares are exchanged (an all-gather here,
    peer stores from inside the kernel there) and added in rank order to the shared expert's rows on every rank, so
    that all ranks hold the same bits for every row and the next layer needs nothing else from the peers.  Returns
    this rank's rows of the last layer's output."""
    import torch
    b_own = x_own.shape[0]
    rows = world * b_own
    x_all = torch.empty((rows, x_own.shape[1]), dtype=x_own.dtype, device=x_own.device)
    dist.all_gather_into_tensor(x_all, x_own.contiguous(), group=group)
    y = None
    for layer in range(layers):
        idx, w = backend.router(layer, x_all)
        share = backend.routed_partial(layer, x_all, idx, w)             # [rows, D] fp32: this rank's experts only
        shares = torch.empty((world * rows, share.shape[1]), dtype=share.dtype, device=share.device)
        dist.all_gather_into_tensor(shares, share.contiguous(), group=group)     # rank r's rows at [r * rows, (r + 1) * rows)
        h1 = backend.shared(layer, x_all)
        y = backend.finalize(shares, h1, world, rows)                            # rank-ordered sum, all rows
        if layer + 1 < layers:
            x_all = backend.renorm(y)
    rank = dist.get_rank(group)
    return y[rank * b_own:(rank + 1) * b_own]


class LibraryBackend:
    """The CUDA library as the arithmetic of the expert-parallel driver.  The handle
    must have been given this rank's expert map and its local blobs per layer."""

    def __init__(self, moe, stream=None):
        import torch
        self.moe, self.torch, self.stream = moe, torch, stream
        c = moe.config
        self.out_dtype = torch.float16 if c.out_dtype == 0 else torch.float32
        self._bufs = {}

    def _buf(self, name, shape, dtype):
        key = (name, tuple(shape), dtype)
        if key not in self._bufs:
            self._bufs[key] = self.torch.empty(shape, dtype=dtype, device="cuda")
        return self._bufs[key]

    def router(self, layer, x_all):
        t, k = x_all.shape[0], self.moe.config.top_k
        idx = self._buf("idx", (t, k), self.torch.int32)
        w = self._buf("w", (t, k), self.torch.float16)
        self.moe.encode_router(layer, x_all, idx, w, tokens=t, stream=self.stream)
        return idx, w

    def routed_partial(self, layer, x_all, idx, w):
        t = x_all.shape[0]
        share = self._buf(("share", layer & 1), (t, self.moe.config.d), self.torch.float32)
        self.moe.routed_partial(layer, x_all, t, idx, w, share, stream=self.stream)
        return share

    def shared(self, layer, x_own):
        if not self.moe.config.shared_f:
            return None
        h1 = self._buf("h1", tuple(x_own.shape), self.out_dtype)
        self.moe.encode_shared_expert(layer, x_own, h1, tokens=x_own.shape[0], stream=self.stream)
        return h1

    def finalize(self, recv, h1, world, b_own):
        y = self._buf("y", (b_own, self.moe.config.d), self.out_dtype)
        self.moe.ep_finalize(recv, world, h1, b_own, y=y, stream=self.stream)
        return y

    def renorm(self, y):
        x = self._buf("xn", tuple(y.shape), self.torch.float16)
        self.moe.rms_renorm(y, y.shape[0], x, stream=self.stream)
        return x
