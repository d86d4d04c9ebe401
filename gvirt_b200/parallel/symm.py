"""Symmetric heap: one slab per rank at identical layout, peer-mapped on every GPU of the group,
plus the Python side of the kernels that use it (stand-alone collectives and the GEMM kernels
that fuse their collective).

The reference's XCCL exports each rank's whole activation pool by IPC key, imports every peer's
pool and uploads a table of peer base pointers plus a flag page (xlite/csrc/ccl.cpp:14-80,
xlite/csrc/kernels/kernel_param.h:8-23); tensors are then named by their offset in the pool.
Same idea here: the slab comes from ``torch.distributed._symmetric_memory`` (cuMem allocation +
handle exchange over the process group), ``peers`` is a device array of the slab base addresses,
and every kernel addresses ``peers[p] + offset``.

*Channels.* A channel is one call site of one collective (e.g. "o_proj all-reduce"): it owns a
flag area, a double-buffered staging / receive area at fixed offsets, and a local two-word state
``{generation, ticket}``. Kernels read the generation from the device, so a captured CUDA graph
can be replayed; two staging parities are enough because a rank can only start launch ``g+2`` of a
channel after it finished ``g+1``, which needed every peer's flags of ``g+1``, which a peer only
sends after its own launch ``g`` — and with it all its reads of parity ``g`` — has completed.
Channels are created in program order, which is identical on all ranks, so offsets match.

*Canaries.* Every region handed out by the heap is followed by a 64-byte guard holding a fixed
pattern that no kernel addresses; ``check_canaries()`` reads the guards back and names the regions
whose guard changed — an overrun by this rank or by a peer's push (the reference has no run-time
race or overrun detection, only static checks; xlite/.clang-tidy:2-40).

With ``world == 1`` (or in single-GPU tests) the heap is an ordinary device buffer and the one
"peer" is the rank itself — the kernels run unchanged.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import torch
import torch.distributed as dist

from .. import _native
from ..config import flags as env_flags

_FLAG_WORDS_PER_CTA = 16
_MAX_GRID = 1024
_GUARD_BYTES = 64
_GUARD_BYTE = 0xA5


@dataclass
class Channel:
    name: str
    flags_off: int
    data_off: int
    data_stride: int   # bytes per parity buffer
    state: torch.Tensor  # local uint32[2]
    grid: int


class SymmetricHeap:
    def __init__(self, group, rank: int, world: int, device: torch.device, nbytes: int = 1 << 30):
        self.group, self.rank, self.world, self.device = group, rank, world, torch.device(device)
        self.nbytes = int(nbytes)
        self.multicast_ptr = 0
        if world > 1:
            import torch.distributed._symmetric_memory as symm_mem
            self.slab = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=self.device)
            self.slab.zero_()
            torch.cuda.synchronize(self.device)
            self.handle = symm_mem.rendezvous(self.slab, group=group)
            ptrs = list(self.handle.buffer_ptrs)
            try:
                self.multicast_ptr = int(self.handle.multicast_ptr or 0)
            except Exception:  # noqa: BLE001 - optional capability
                self.multicast_ptr = 0
            dist.barrier(group=group)
        else:
            self.slab = torch.zeros(self.nbytes, dtype=torch.uint8, device=self.device)
            self.handle = None
            ptrs = [self.slab.data_ptr()]
        assert ptrs[rank] == self.slab.data_ptr()
        self.peer_ptrs = ptrs
        self.peers = torch.tensor(ptrs, dtype=torch.int64, device=self.device)
        self._cursor = 0
        self._guards: list = []   # (offset, label) of every guard, in allocation order
        self.channels: Dict[str, Channel] = {}
        self._ag_maps: Dict[str, torch.Tensor] = {}
        props = torch.cuda.get_device_properties(self.device)
        self.num_sms = props.multi_processor_count
        # fused GEMM + all-reduce: at 8 ranks a tile is reduced by one owner rank and the result
        # broadcast (two hops, 2 (R - 1) / R of a message per rank) instead of everyone sending
        # everything to everyone (one hop, R - 1 messages per rank); up to 4 ranks the single hop
        # wins (Llama-3-8B decode at TP4: 21.5 k tok/s one hop, 20.9 k two hops)
        import os
        mode = os.environ.get("GVIRT_AR_TWO_SHOT", "")
        self.ar_two_shot = (world > 4) if mode == "" else mode not in ("0", "false", "off")

    # ------------------------------------------------------------------ layout
    def _take(self, nbytes: int, align: int = 1024, label: str = "") -> int:
        off = (self._cursor + align - 1) // align * align
        if off + nbytes + _GUARD_BYTES > self.nbytes:
            raise RuntimeError(f"symmetric heap exhausted: need {nbytes} bytes at {off}, size {self.nbytes}")
        self._cursor = off + nbytes + _GUARD_BYTES
        # the guard lives in this rank's slab only; peers never address it
        self.slab[off + nbytes: off + nbytes + _GUARD_BYTES].fill_(_GUARD_BYTE)
        self._guards.append((off + nbytes, label or f"region@{off}"))
        return off

    def check_canaries(self) -> list:
        """Labels of the regions whose trailing guard no longer holds the pattern (empty = intact).
        One small device-to-host read; meant for tests, the paranoid debug mode and post-mortems."""
        if not self._guards:
            return []
        idx = torch.tensor([g[0] for g in self._guards], dtype=torch.long, device=self.device)
        span = idx.unsqueeze(1) + torch.arange(_GUARD_BYTES, device=self.device)
        ok = (self.slab[span] == _GUARD_BYTE).all(dim=1).cpu().tolist()
        return [label for (_, label), good in zip(self._guards, ok) if not good]

    def channel(self, name: str, data_bytes: int, grid: int) -> Channel:
        """Create (or fetch) a channel with `data_bytes` per parity buffer."""
        ch = self.channels.get(name)
        if ch is not None:
            if ch.data_stride < data_bytes or ch.grid < grid:
                raise RuntimeError(f"channel {name} was created smaller than now requested")
            return ch
        flags_off = self._take(2 * _MAX_GRID * _FLAG_WORDS_PER_CTA * 4, label=f"{name}/flags")
        stride = (data_bytes + 1023) // 1024 * 1024
        data_off = self._take(2 * stride, label=f"{name}/data")
        state = torch.zeros(2, dtype=torch.int32, device=self.device)
        ch = Channel(name, flags_off, data_off, stride, state, grid)
        self.channels[name] = ch
        return ch

    # ------------------------------------------------------------------ capability checks
    def supports(self, x: torch.Tensor) -> bool:
        # bandwidth-bound sizes go to the library: these kernels are built for latency
        return (x.is_cuda and x.dtype in (torch.bfloat16, torch.float32) and x.is_contiguous()
                and x.data_ptr() % 16 == 0 and x.numel() * x.element_size() <= env_flags().symm_max_bytes
                and not env_flags().disable_symm)

    def can_fuse_gemm_ar(self, x: torch.Tensor, w: torch.Tensor) -> bool:
        M = x.numel() // x.shape[-1]
        N = w.shape[0]
        return (not env_flags().disable_symm and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
                and 0 < M <= 128
                and N % 8 == 0 and (N + 127) // 128 <= 2 * self.num_sms and x.shape[-1] % 8 == 0
                and self.world <= 8)

    def can_fuse_gemm_rs(self, x: torch.Tensor, w: torch.Tensor) -> bool:
        M, N = x.shape[0], w.shape[0]
        return (not env_flags().disable_symm and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
                and M % (128 * self.world) == 0
                and N % 16 == 0 and x.shape[1] % 8 == 0 and M // self.world <= self.sp_rows_cap)

    def can_fuse_ag_gemm(self, x_local: torch.Tensor, w: torch.Tensor) -> bool:
        m_r = x_local.shape[0]
        return (not env_flags().disable_symm and x_local.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
                and m_r % 128 == 0 and w.shape[0] % 8 == 0
                and x_local.shape[1] % 8 == 0 and m_r <= self.sp_rows_cap and x_local.is_contiguous())

    # ------------------------------------------------------------------ sequence-parallel fused GEMMs
    sp_rows_cap = 2048  # token rows per rank the receive / staging regions are sized for

    def gemm_reduce_scatter(self, x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None):
        """out[M / R, N] = reduce_scatter(x_shard @ w_shard^T); see csrc/kernels/gemm_sp.cu."""
        M, K = x.shape
        N = w.shape[0]
        R = self.world
        if out is None:
            out = torch.empty(M // R, N, dtype=x.dtype, device=x.device)
        cap = self.sp_rows_cap
        ch = self.channel(f"gemm_rs:{N}", R * cap * N * 2, 1)
        _native.call("gemm_rs", x, w, out, M, N, K, x.stride(0), w.stride(0), out.stride(0), self.peers,
                     ch.data_off, ch.data_stride, ch.flags_off, ch.state, self.rank, R, cap)
        return out

    def allgather_gemm(self, x_local: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None,
                       bias: Optional[torch.Tensor] = None):
        """out[M, N] = all_gather(x_local)[M, K] @ w^T (+ bias); see csrc/kernels/gemm_sp.cu."""
        m_r, K = x_local.shape
        N = w.shape[0]
        R = self.world
        M = m_r * R
        if out is None:
            out = torch.empty(M, N, dtype=x_local.dtype, device=x_local.device)
        cap = self.sp_rows_cap
        name = f"ag_gemm:{K}"
        fresh = name not in self.channels
        ch = self.channel(name, R * cap * K * 2, 1)      # one slot per source rank and parity
        if fresh:
            import ctypes
            maps = torch.empty(2 * R * 128, dtype=torch.uint8, device=self.device)
            host_peers = (ctypes.c_longlong * R)(*self.peer_ptrs)
            _native.call("ag_gemm_setup", maps, host_peers, ch.data_off, ch.data_stride, cap, K, R, self.rank)
            self._ag_maps[name] = maps
        _native.call("ag_gemm", x_local, w, bias, out, M, N, K, w.stride(0), out.stride(0), self._ag_maps[name],
                     self.peers, ch.data_off, ch.data_stride, ch.flags_off, ch.state, self.rank, R, cap)
        return out

    # ------------------------------------------------------------------ collectives
    def _grid_for(self, nbytes: int) -> int:
        # one CTA per ~32 KiB, at most one per SM; must be identical on every rank (it is: the
        # payload size is)
        return max(1, min(self.num_sms, (nbytes + 32767) // 32768))

    def _coll(self, mode: int, x: torch.Tensor, out: torch.Tensor, n: int, stage_elems: int, tag: str):
        esz = x.element_size()
        nbytes = stage_elems * esz
        # channels are bucketed by power-of-two capacity so that a handful serve all sizes
        cap = 1 << max(16, (nbytes - 1).bit_length())
        ch = self.channel(f"{tag}:{cap}", cap, self.num_sms)
        grid = self._grid_for(n * esz)
        _native.call("collective", mode, int(x.dtype == torch.float32), x, out, n, self.peers,
                     ch.flags_off, ch.data_off, ch.data_stride, ch.state, self.rank, self.world, grid)
        return out

    ll_max_bytes = 1 << 20  # per-slice payload up to which the push (flag-in-data) kernels are used

    def _coll_ll(self, mode: int, x: torch.Tensor, out: torch.Tensor, n: int, tag: str):
        """Low-latency push form of modes 0 / 1 / 2 (kernel modes 4 / 5 / 6): n elements per slice."""
        esz = x.element_size()
        lines = n * esz // 8
        cap_lines = 1 << max(10, (lines - 1).bit_length())
        ch = self.channel(f"{tag}:{cap_lines}", 16 * (self.world + 1) * cap_lines, 1)
        grid = max(1, min(self.num_sms, (lines + 511) // 512))
        if mode == 0 and self.ar_two_shot and self.world > 1:
            mode = 3          # kernel mode 7: owner-reduces-and-broadcasts all-reduce
        _native.call("collective", mode + 4, int(x.dtype == torch.float32), x, out, n, self.peers,
                     ch.flags_off, ch.data_off, ch.data_stride, ch.state, self.rank, self.world, grid)
        return out

    def _use_ll(self, n: int, esz: int) -> bool:
        return (n * esz) % 8 == 0 and n * esz <= self.ll_max_bytes

    def all_reduce(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Sum over the group (in place unless `out` is given). One-shot below 512 KiB, two-shot
        (reduce-scatter + all-gather) above when the size divides evenly."""
        out = x if out is None else out
        n = x.numel()
        esz = x.element_size()
        R = self.world
        if self._use_ll(n, esz):
            return self._coll_ll(0, x, out, n, "ar_ll")
        if n * esz > (512 << 10) and n % R == 0 and ((n // R) * esz) % 16 == 0:
            return self._coll(3, x, out, n // R, 2 * n, "ar2")
        return self._coll(0, x, out, n, n, "ar1")

    def all_gather(self, x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        n = x.numel()
        if (n * x.element_size()) % 16:
            dist.all_gather_into_tensor(out, x, group=self.group)
            return out
        if self._use_ll(n, x.element_size()):
            return self._coll_ll(1, x, out, n, "ag_ll")
        return self._coll(1, x, out, n, n, "ag")

    def reduce_scatter(self, x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        n = x.numel() // self.world
        if (n * x.element_size()) % 16:
            dist.reduce_scatter_tensor(out, x, group=self.group)
            return out
        if self._use_ll(n, x.element_size()):
            return self._coll_ll(2, x, out, n, "rs_ll")
        return self._coll(2, x, out, n, x.numel(), "rs")

    # ------------------------------------------------------------------ fused GEMM + all-reduce
    def gemm_allreduce(self, x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None,
                       bias: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None,
                       tag: Optional[str] = None, ss_out: Optional[torch.Tensor] = None,
                       next_w: Optional[torch.Tensor] = None) -> torch.Tensor:
        """out = sum_r x_r @ w_r^T (+ bias) (+ residual); see csrc/kernels/gemm_allreduce.cu.
        `out` may be `residual` itself (the residual stream updated in place); `ss_out` fp32
        [tokens, N / 128] receives the sums of squares of the new rows per 128-feature tile."""
        x2 = x.reshape(-1, x.shape[-1])
        M, K = x2.shape
        N = w.shape[0]
        if out is None:
            out = torch.empty(*x.shape[:-1], N, dtype=x.dtype, device=x.device)
        o2 = out.reshape(-1, N)
        m_cap = 128
        name = tag or f"gemm_ar:{N}x{K}"
        # receive region per parity: [R sources + 1 final][m_cap tokens][N / 4] sixteen-byte lines
        ch = self.channel(name, (self.world + 1) * m_cap * N * 4, 2 * self.num_sms)
        if next_w is not None:
            from ..ops.decode_ops import _hint_next
            _hint_next(next_w)          # this launch warms L2 with the first tiles of the GEMM behind it
        _native.call("gemm_allreduce_ss", x2, w, bias, residual, o2, ss_out,
                     ss_out.stride(0) if ss_out is not None else 0, M, N, K, x2.stride(0), w.stride(0),
                     o2.stride(0), self.peers, ch.data_off, ch.flags_off, ch.state, self.rank, self.world,
                     m_cap, 2 * self.num_sms, int(self.ar_two_shot))
        return out


def group_is_single_node(ranks, devs_per_node: int) -> bool:
    """Peer mapping needs NVLink: a group whose global ranks fall on more than one node (ranks are
    laid out node by node, `devs_per_node` per node) keeps the library backend, like the reference
    enables its own collectives intra-node only (xlite/csrc/runtime.cpp:228-278)."""
    return len({r // max(devs_per_node, 1) for r in ranks}) <= 1


def attach_symmetric_heap(ctx, nbytes: int = 1 << 30, ep_nbytes: int = 0) -> None:
    """Create the TP-group heap (and, for expert parallelism, the EP-group heap) on `ctx`."""
    if ctx.device.type != "cuda" or env_flags().disable_symm:
        return
    dpn = env_flags().devs_per_node
    if not group_is_single_node(ctx.tp_ranks(), dpn):
        nbytes = 0
    if not group_is_single_node(ctx.ep_ranks(), dpn):
        ep_nbytes = 0
    shared = (ctx.tp > 1 and nbytes > 0 and ctx.ep > 1 and ep_nbytes > 0
              and (ctx.ep_group is ctx.tp_group or ctx.ep == ctx.tp))
    if ctx.tp > 1 and nbytes > 0:
        # experts spread over the same ranks as the tensor-parallel group: one heap serves both
        ctx.symm = SymmetricHeap(ctx.tp_group, ctx.tp_rank, ctx.tp, ctx.device,
                                 nbytes + (ep_nbytes if shared else 0))
    if ctx.ep > 1 and ep_nbytes > 0:
        if shared:
            ctx.symm_ep = ctx.symm
        else:
            ctx.symm_ep = SymmetricHeap(ctx.ep_group, ctx.ep_rank, ctx.ep, ctx.device, ep_nbytes)
