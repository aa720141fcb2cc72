"""`Buffer`: expert-parallel dispatch / combine over NVLink peer memory, and the
`StreamingHandle` that carries one dispatch's state.

Public surface and semantics follow the reference (stream_ep/buffer.py:14-782):
``Buffer(group, num_nvl_bytes, ...)``, ``dispatch`` / ``dispatch_grads`` /
``combine`` / ``combine_grads``, the launch-gate helpers, ``set_num_sms`` and the
``get_*_config`` tables.  The transport underneath is different: there are no
ring buffers and no receiver kernels.  Every rank maps every peer's *symmetric
arena*; dispatch pushes each token row directly into its final, expert-major,
128-row-padded pool slot in the owner's HBM and release-adds the owner's
per-tile arrival counter; combine pulls the partial rows back and reduces them
in fp32.  The layer-level fused kernels (see ``stream_moe``) reuse the same
records and counters.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Any, List, Optional, Sequence, Tuple

import torch

from . import _ext
from .errors import StreamEPError, StreamEPOverflow, StreamEPTimeout

topk_idx_t = torch.int64

# launch-gate ids of the native runtime
_GATE_DISPATCH, _GATE_DISPATCH_GRADS, _GATE_KERNEL_Y, _GATE_KERNEL_A_BWD = 0, 1, 2, 3


def _C():
    return _ext.load()


def __getattr__(name):  # Config / EventHandle live in the native module
    if name in ("Config", "EventHandle"):
        return getattr(_C(), name)
    raise AttributeError(name)


@dataclass
class StreamingHandle:
    """All per-dispatch state (reference: stream_ep/buffer.py:14-95, same field
    names and meanings).

    Pool layout: rows are expert-major; expert ``e`` owns rows
    ``[expert_pool_block_offset[e] * tile_m, expert_pool_block_offset[e+1] * tile_m)``
    of which the first ``expert_frequency[e]`` are valid; padding rows have
    ``pool_recv_token == -1``.
    """
    pool: torch.Tensor                        # [TK_padded, hidden] bf16
    pool_topk_weight: torch.Tensor            # [TK_padded] f32
    pool_recv_token: torch.Tensor             # [TK_padded] i32 (-1 = padding)
    pool_k_slot: torch.Tensor                 # [TK_padded] i32 (-1 = padding)
    send_head: torch.Tensor                   # [T, R] i32, gap-encoded stream positions
    is_token_in_rank: torch.Tensor            # [T, R] bool
    rank_prefix_matrix: torch.Tensor          # [R, R] i32 (own column)
    channel_prefix_matrix: torch.Tensor       # [R, C] i32
    recv_channel_prefix_matrix: torch.Tensor  # [R, C] i32
    expert_frequency: torch.Tensor            # [E_local] i32
    expert_pool_block_offset: torch.Tensor    # [E_local + 1] i32 (tile units)
    base_pool: torch.Tensor                   # [C, R, E_local] i32
    seen_per_substream: torch.Tensor          # [C, R, E_local] i32
    tile_id_to_expert: torch.Tensor           # [total_tiles] i32
    pool_arrival_target: torch.Tensor         # [total_tiles] i32
    pool_arrival_count: torch.Tensor          # [total_tiles] i32
    k_local_remaining: torch.Tensor           # [T_recv] i32
    y_done_per_token: torch.Tensor            # [T_recv] i64
    o: torch.Tensor                           # [T_recv, hidden] bf16, zero
    recv_token_to_slots: torch.Tensor         # [T_recv, K] i32 (-1 = other rank)
    k_local_total: torch.Tensor               # [T_recv] i32
    total_tiles: int
    tile_m: int
    TK_padded: int
    dispatch_seq: int
    # native per-dispatch state: sender-side routing (destination slot of every pair, recv-token
    # id of every token at every rank) and the per-slot source table used by the fused combine
    _dispatch_out: Any = None

    # Aliases in the wording of the reference's README (tile_ready / a_ready): a tile is ready when
    # its arrival count equals its target.
    @property
    def tile_ready(self) -> torch.Tensor:
        return self.pool_arrival_count == self.pool_arrival_target

    @property
    def pool_src(self) -> torch.Tensor:
        """[TK_padded, 2] i32: (source rank, source token) of every slot (-1 = padding)."""
        return self._dispatch_out.pool_src

    @property
    def num_recv_tokens(self) -> int:
        return self._dispatch_out.num_recv_tokens

    def stats(self, rank: Optional[int] = None) -> dict:
        """Per-dispatch counters for logging (synchronises: it reads device tensors).

        ``pairs_received`` / ``recv_tokens`` / ``total_tiles`` / ``padding_ratio`` describe this
        rank's pool; ``pairs_sent_remote`` and the byte counts describe what this rank's push
        (dispatch: one row per pair) and the matching combine traffic (one row per pair back to
        the source) move over NVLink.  ``rank`` (this rank's index) is needed for the remote counts."""
        hidden = int(self.pool.shape[1]) if self.pool.dim() == 2 else 0
        freq = self.expert_frequency.cpu()
        pairs = int(freq.sum())
        out = {"pairs_received": pairs, "recv_tokens": self.num_recv_tokens, "total_tiles": int(self.total_tiles),
               "rows_padded": int(self.TK_padded),
               "padding_ratio": (self.TK_padded - pairs) / self.TK_padded if self.TK_padded else 0.0,
               "max_expert_rows": int(freq.max()) if freq.numel() else 0, "dispatch_seq": int(self.dispatch_seq)}
        if rank is not None and self._dispatch_out is not None:
            idx = self._dispatch_out.topk_idx
            el = max(self._dispatch_out.num_experts // max(int(self.is_token_in_rank.shape[1]), 1), 1)
            remote = int(((idx >= 0) & (idx // el != rank)).sum())
            out.update(pairs_sent_remote=remote, dispatch_bytes_out=remote * hidden * 2,
                       combine_bytes_in=remote * hidden * 2)
        return out


class Buffer:
    """Symmetric-memory communication buffer for one expert-parallel group.

    Arguments follow stream_ep/buffer.py:125-151.  ``num_nvl_bytes`` sizes the
    symmetric arena: unlike the reference's ring buffers, the arena holds the
    pools, per-slot arrays and outputs that peers write into, so it must cover
    what all layers keep alive between forward and backward (see
    ``Buffer.get_arena_size_hint``).  ``num_rdma_bytes`` must be 0: the RDMA
    path is out of scope on one NVSwitch domain.
    """

    num_sms: int = 80
    _num_sms_explicit: bool = False

    def __init__(self, group, num_nvl_bytes: int = 0, num_rdma_bytes: int = 0,
                 allow_mnnvl: bool = False, use_fabric: bool = False,
                 explicitly_destroy: bool = False, enable_shrink: bool = False,
                 comm=None, *, timeout_ms: Optional[int] = None, allocator: Optional[str] = None,
                 _local: Optional[Tuple["LocalWorld", int]] = None) -> None:
        import torch.distributed as dist

        if num_rdma_bytes:
            raise StreamEPError("the internode (RDMA) path is not available: one NVSwitch domain only")
        if allow_mnnvl:
            raise StreamEPError("allow_mnnvl: multi-node NVLink domains are not supported (one NVSwitch domain of up to 8 GPUs)")
        if enable_shrink:
            raise StreamEPError("enable_shrink is not supported (the reference allocates its mask buffers but no kernel "
                                "reads them: csrc/stream_ep.cpp:526-533); use Buffer.recover() after a failed collective")
        # Two allocators for the symmetric arena (reference: SharedMemoryAllocator, csrc/stream_ep.cpp:52-124):
        # "ipc" = cudaMalloc + CUDA IPC handles, "vmm" = cuMemCreate + POSIX file descriptors + cuMemMap.  The
        # reference's `use_fabric` asks for its second (VMM) allocator with fabric handles; inside one node the
        # shareable handle is a file descriptor, so `use_fabric=True` selects "vmm" here.
        if allocator is None:
            allocator = os.environ.get("STREAM_EP_ALLOCATOR", "vmm" if use_fabric else "ipc")
        if allocator not in ("ipc", "vmm"):
            raise ValueError(f"allocator must be 'ipc' or 'vmm', got {allocator!r}")
        self.allocator = allocator
        self._local = _local
        if _local is not None:
            world, rank = _local
            self.rank, self.group_size, self.group = rank, world.num_ranks, world
            all_gather_object = None
        elif group is not None:
            self.rank, self.group_size, self.group = group.rank(), group.size(), group

            def all_gather_object(obj):
                out = [None] * self.group_size
                dist.all_gather_object(out, obj, group)
                return out
        elif comm is not None:
            self.rank, self.group_size, self.group = comm.Get_rank(), comm.Get_size(), comm

            def all_gather_object(obj):
                return comm.allgather(obj)
        else:
            raise ValueError("Either 'group' or 'comm' must be provided.")
        if self.group_size not in (1, 2, 4, 8):
            raise StreamEPError(f"unsupported number of EP ranks: {self.group_size} (1, 2, 4 or 8)")
        Buffer.autopick_num_sms(self.group_size)
        from .utils.nvlink import check_nvlink_connections
        if _local is None:
            check_nvlink_connections(group if group is not None else comm)

        self.num_nvl_bytes = int(num_nvl_bytes)
        self.num_rdma_bytes = 0
        self.explicitly_destroy = explicitly_destroy
        self.enable_shrink = enable_shrink
        self.num_channels = max(1, min(Buffer.num_sms // 2, _C().MAX_CHANNELS))
        if timeout_ms is None:
            timeout_ms = int(os.environ.get("STREAM_EP_TIMEOUT_MS", "10000"))
        arena_bytes = self.num_nvl_bytes if self.num_nvl_bytes > 0 else int(
            os.environ.get("STREAM_EP_ARENA_BYTES", str(2 << 30)))
        self.runtime = _C().Runtime(self.rank, self.group_size, arena_bytes, self.num_channels,
                                    _C().MAX_EXPERTS, timeout_ms, allocator == "vmm")
        if _local is None:
            device_ids = all_gather_object(self.runtime.get_local_device_id())
            if allocator == "vmm" and self.group_size > 1:
                self._sync_vmm(all_gather_object)
            else:
                handles = all_gather_object(self.runtime.get_local_ipc_handle()
                                            if self.group_size > 1 and allocator == "ipc" else None)
                self.runtime.sync(device_ids, handles)
            assert self.runtime.is_available()
        self._next_seq = 0
        self._push_blocks = 0  # 0 = auto
        self._compute_stream_handle = None
        self._default_stream_handle = None
        chunk = os.environ.get("STREAM_EP_PUSH_CHUNK_PAIRS")
        if chunk:
            self.runtime.set_pairs_per_chunk(int(chunk))
        order = os.environ.get("STREAM_EP_PUSH_ORDER")
        if order:
            self.runtime.set_push_order(int(order))
        warps = os.environ.get("STREAM_EP_PUSH_WARPS")
        if warps:
            self.runtime.set_active_push_warps(int(warps))
        ctas = os.environ.get("STREAM_EP_PUSH_CTAS")
        if ctas:
            self.runtime.set_push_ctas(int(ctas))
        split = os.environ.get("STREAM_EP_SPLIT_LOCAL")
        if split:
            self.runtime.set_split_local(split not in ("0", "false", "False"))
        bulk = os.environ.get("STREAM_EP_BULK_PUSH")
        if bulk:
            self.runtime.set_bulk_push(bulk not in ("0", "false", "False"))

    def _sync_vmm(self, all_gather_object) -> None:
        """Hand every peer a file descriptor of this rank's arena allocation and map theirs.  Descriptors cross
        process boundaries as SCM_RIGHTS messages on Unix sockets in the abstract namespace: every rank listens on
        a name derived from a token that rank 0 draws, sends its descriptor to whoever connects, and connects to
        every peer in turn."""
        import socket
        import threading
        import uuid

        token = all_gather_object(uuid.uuid4().hex if self.rank == 0 else None)[0]
        name = lambda r: f"\0streamep_b200_{token}_{r}"   # noqa: E731
        fd = self.runtime.export_vmm_fd()
        srv = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        srv.bind(name(self.rank))
        srv.listen(self.group_size)
        srv.settimeout(60)

        def serve():
            for _ in range(self.group_size - 1):
                conn, _addr = srv.accept()
                with conn:
                    socket.send_fds(conn, [b"fd"], [fd])
        th = threading.Thread(target=serve, daemon=True)
        th.start()
        sizes = all_gather_object(self.runtime.arena_total_bytes())     # also: every rank is listening by now
        fds = [-1] * self.group_size
        try:
            for r in range(self.group_size):
                if r == self.rank:
                    continue
                with socket.socket(socket.AF_UNIX, socket.SOCK_STREAM) as c:
                    c.settimeout(60)
                    c.connect(name(r))
                    _msg, got, _flags, _addr = socket.recv_fds(c, 16, 1)
                    if len(got) != 1:
                        raise StreamEPError(f"rank {self.rank}: no file descriptor received from rank {r}")
                    fds[r] = got[0]
            self.runtime.sync_vmm(fds, [int(v) for v in sizes])
        finally:
            th.join(timeout=60)
            srv.close()
            for f in fds + [fd]:
                if f >= 0:
                    os.close(f)

    # ------------------------------------------------------------------ lifecycle
    def destroy(self):
        assert self.explicitly_destroy, "`explicitly_destroy` flag must be set"
        self.runtime.destroy()
        self.runtime = None

    def state_dict(self) -> dict:
        """The only state that matters across iterations is the sequence counter
        (stream_ep/buffer.py:255-261); a resumed process builds a fresh Buffer."""
        return {"next_seq": self._next_seq}

    def load_state_dict(self, state: dict) -> None:
        self._next_seq = int(state["next_seq"])

    # ------------------------------------------------------------------ failure reporting
    def check_status(self) -> None:
        """Synchronise the device and raise :class:`StreamEPTimeout` if any bounded
        device wait gave up since the last check (:class:`StreamEPOverflow` if a
        capacity-mode dispatch did not fit its region).  The context stays usable."""
        msg = self.runtime.poll_status(True)
        if msg:
            if "capacity overflow" in msg:
                raise StreamEPOverflow(f"rank {self.rank}: {msg}; {self._overflow_text()}")
            raise StreamEPTimeout(f"rank {self.rank}: {msg}")

    # ------------------------------------------------------------------ capacity mode
    def enable_capacity_mode(self, max_tokens: int, hidden: int, num_topk: int, num_experts: int, *,
                             capacity_factor: float = 1.5, layers_in_flight: int = 1) -> None:
        """Switch the fused layer (``stream_moe_func``) of this buffer to fixed receive regions, which removes
        the host read of the receive sizes from every forward (the reference pays the same read:
        csrc/stream_ep.cpp:741-759).

        Collective: every rank calls it once, right after constructing the buffer, with the same arguments.
        Each of the ``layers_in_flight`` regions holds a pool of ``capacity_factor x max_tokens x num_topk``
        rows (the balanced load is ``max_tokens x num_topk``) plus one padding tile per local expert.  Kernels
        then take the live sizes from device memory; a dispatch whose layout exceeds the capacity on any rank
        is run as an EMPTY dispatch by all ranks (they all see the same counts), recorded in the status block
        and in ``overflow_info()``, and reported by ``check_status()`` as :class:`StreamEPOverflow` - i.e. one
        step late, without a device sync in the step itself.  Dispatches whose shape differs from the
        configured one (more tokens, another hidden size or top-k) keep using exactly sized buffers.
        The stand-alone ``dispatch`` keeps exact sizing unless called with ``capacity_mode=True``."""
        import torch.distributed as dist

        R = self.group_size
        el = max(num_experts // R, 1)
        rows = int(max_tokens * num_topk * capacity_factor) + 128 * el
        rows_cap = (rows + 127) // 128 * 128
        recv_cap = min(max_tokens * R, rows_cap)
        base = self.runtime.enable_static(int(layers_in_flight), int(max_tokens), int(hidden), int(num_topk),
                                          int(rows_cap), int(recv_cap))
        # the regions must sit at the same arena offset on every rank
        if self._local is not None:
            world = self._local[0]
            world._static_bases[self.rank] = base
            if all(b is not None for b in world._static_bases) and len(set(world._static_bases)) != 1:
                raise StreamEPError(f"capacity-mode regions ended up at different arena offsets: {world._static_bases}")
        elif R > 1:
            every = [None] * R
            dist.all_gather_object(every, base, self.group)
            if len(set(every)) != 1:
                raise StreamEPError(f"capacity-mode regions ended up at different arena offsets: {every}; "
                                    "call enable_capacity_mode right after constructing the Buffer on every rank")
            dist.barrier(self.group)

    @staticmethod
    def capacity_mode_bytes(max_tokens: int, hidden: int, num_topk: int, num_experts: int, num_ranks: int, *,
                            capacity_factor: float = 1.5, layers_in_flight: int = 1) -> int:
        """Arena bytes :meth:`enable_capacity_mode` takes for these arguments (add them to ``num_nvl_bytes``)."""
        el = max(num_experts // num_ranks, 1)
        rows = (int(max_tokens * num_topk * capacity_factor) + 128 * el + 127) // 128 * 128
        recv = min(max_tokens * num_ranks, rows)
        region = rows * hidden * 2 + rows * 20 + recv * (num_topk * 4 + 24) + rows // 128 * 4 + 16 * 1024
        grads = 2 * (rows * hidden * 2 + rows // 128 * 4 + 2048)
        landing = 2 * max_tokens * num_topk * hidden * 2 if num_ranks > 1 else 0
        dwt = 2 * (max_tokens * num_topk * 4 + 1024)
        return int(layers_in_flight * region + grads + landing + dwt + (1 << 20))

    @property
    def capacity_mode(self) -> bool:
        return self.runtime is not None and self.runtime.static_enabled()

    def overflow_info(self) -> dict:
        """Capacity-mode overflow record, read from pinned host memory (no device sync): how many dispatches
        overflowed so far and what the last one would have needed."""
        c, epoch, tiles, recv = self.runtime.overflow_info()
        return {"count": int(c), "epoch": int(epoch), "needed_tiles": int(tiles), "needed_recv_tokens": int(recv)}

    def _overflow_text(self) -> str:
        info, cap = self.overflow_info(), self.runtime.static_capacity()
        if not cap:
            return ""
        return (f"needed {info['needed_tiles']} tiles / {info['needed_recv_tokens']} recv tokens on the fullest rank, "
                f"capacity is {cap[2] // 128} tiles / {cap[3]} recv tokens: raise capacity_factor")

    def set_timeout_ms(self, ms: int) -> None:
        self.runtime.set_timeout_ms(int(ms))

    def recover(self) -> None:
        """Collective host-side recovery after a failed collective (a rank that did not
        join, a wait that ran out).  Every rank of the group must call it: the device is
        drained, the status block cleared, and the per-kind epoch counters - which went
        out of step when only some ranks launched the failed operation - are re-agreed
        as the maximum over the group.  Tensors of the failed operation must not be used."""
        import torch.distributed as dist

        torch.cuda.synchronize()
        self.runtime.poll_status(True)
        mine = self.runtime.get_epochs()
        if self._local is not None:
            every = [b.runtime.get_epochs() for b in self._local[0].buffers]
        else:
            every = [None] * self.group_size
            dist.all_gather_object(every, mine, self.group)
        agreed = [max(col) + 2 for col in zip(*every)]
        self.runtime.set_epochs(agreed)
        self.runtime.static_reset()      # capacity mode: the alternating regions start over on every rank
        if self._local is None and self.group_size > 1:
            dist.barrier(self.group)

    # ------------------------------------------------------------------ symmetric memory
    def alloc_symmetric(self, shape: Sequence[int], dtype: torch.dtype, zero: bool = False) -> torch.Tensor:
        """A tensor in the peer-mapped arena.  Gates and rows that peers read while they
        are still being produced (``o``, ``y_done_per_token``, ``dL_dx_per_r``,
        ``bwd_a_done_per_token``) must live here; the block returns to the arena when
        the tensor is garbage collected."""
        return self.runtime.alloc_symmetric(list(shape), dtype, zero)

    def get_local_buffer_tensor(self, dtype: torch.dtype, size: Optional[torch.Size] = None,
                                offset: int = 0, use_rdma_buffer: bool = False) -> torch.Tensor:
        """API parity with stream_ep/buffer.py:381-400: a scratch tensor in the arena."""
        assert not use_rdma_buffer, "no RDMA buffer on one NVSwitch domain"
        numel = size.numel() if size is not None else 1024
        t = self.alloc_symmetric([offset + numel], dtype)
        t = t[offset:]
        return t if size is None else t.view(size)

    @staticmethod
    def get_arena_size_hint(num_tokens: int, hidden: int, num_topk: int, num_ranks: int,
                            num_local_experts: int, layers_in_flight: int = 1,
                            imbalance: float = 1.5) -> int:
        """Bytes of symmetric memory for ``layers_in_flight`` layers (forward state
        kept until backward) plus one backward's transients."""
        per_layer = _C().layer_bytes_hint(num_tokens, hidden, num_topk, num_ranks, num_local_experts, imbalance)
        return int(per_layer * (layers_in_flight + 1.5))

    # ------------------------------------------------------------------ launch gates
    def local_phase_event(self):
        """``EventHandle`` recorded where the most recent backward finished its last kernel that talks to
        peers (what follows are the local dW GEMMs), or ``None`` before the first backward.  A loader that
        makes its host-to-device copy of the next batch wait on it (``copy_stream.wait_event(ev)``) overlaps
        the copy with local compute only: kernels that synchronise with peers at system scope measured up to
        4x slower while a PCIe copy was in flight."""
        return self.runtime.local_phase_event()

    def set_compute_stream_handle(self, stream) -> None:
        """Remember the caller's compute stream (reference: csrc/stream_ep.cpp:387-456, called from
        stream_ep/stream_moe/stream_moe.py:1239).  The gate helpers wait on it when no stream is given."""
        self._compute_stream_handle = stream

    def set_default_stream_handle(self, stream) -> None:
        """Remember the stream the layer was called on (stream_ep/stream_moe/stream_moe.py:1247)."""
        self._default_stream_handle = stream

    def _raw(self, stream):
        if stream is None:
            stream = self._compute_stream_handle if self._compute_stream_handle is not None else torch.cuda.current_stream()
        return stream.cuda_stream

    def wait_dispatch_main_started(self, stream=None) -> None:
        """Hold ``stream`` at the GPU front-end until the last dispatch kernel is resident
        (reference: stream_ep/buffer.py:274-284)."""
        self.runtime.gate_wait_started(_GATE_DISPATCH, self._raw(stream))

    def wait_dispatch_grads_started(self, stream=None) -> None:
        self.runtime.gate_wait_started(_GATE_DISPATCH_GRADS, self._raw(stream))

    def wait_kernel_y_started(self, stream=None) -> None:
        self.runtime.gate_wait_started(_GATE_KERNEL_Y, self._raw(stream))

    def wait_kernel_a_bwd_started(self, stream=None) -> None:
        self.runtime.gate_wait_started(_GATE_KERNEL_A_BWD, self._raw(stream))

    def bump_kernel_y_issued(self) -> None:
        self.runtime.gate_bump_issued(_GATE_KERNEL_Y)

    def bump_kernel_a_bwd_issued(self) -> None:
        self.runtime.gate_bump_issued(_GATE_KERNEL_A_BWD)

    def kernel_y_started_flag_view(self) -> torch.Tensor:
        return self.runtime.gate_flag_tensor(_GATE_KERNEL_Y)

    def kernel_a_bwd_started_flag_view(self) -> torch.Tensor:
        return self.runtime.gate_flag_tensor(_GATE_KERNEL_A_BWD)

    # ------------------------------------------------------------------ config policy
    @staticmethod
    def is_sm90_compiled() -> bool:
        return False

    @staticmethod
    def is_sm100_compiled() -> bool:
        return bool(_C().is_sm100_compiled())

    @staticmethod
    def set_num_sms(new_num_sms: int) -> None:
        assert new_num_sms % 2 == 0, "The SM count must be even"
        Buffer.num_sms = new_num_sms
        Buffer._num_sms_explicit = True

    @staticmethod
    def autopick_num_sms(group_size: int) -> int:
        """80 for one or two nodes, 64 beyond (stream_ep/buffer.py:363-379).  Here the
        value sets the number of channels (num_sms // 2) of the deterministic pool
        layout and the grid of the stand-alone push / pull kernels."""
        if not Buffer._num_sms_explicit:
            nodes = (group_size + 7) // 8
            Buffer.num_sms = 80 if nodes <= 2 else 64
        return Buffer.num_sms

    @staticmethod
    def get_dispatch_config(num_ranks: int):
        Buffer.autopick_num_sms(num_ranks)
        table = {1: (24, 256), 2: (24, 256), 4: (6, 256), 8: (6, 256)}
        assert num_ranks in table, f"Unsupported number of EP ranks: {num_ranks}"
        s, r = table[num_ranks]
        return _C().Config(Buffer.num_sms, s, r, 6, 128)

    @staticmethod
    def get_combine_config(num_ranks: int):
        Buffer.autopick_num_sms(num_ranks)
        table = {1: (10, 256), 2: (10, 256), 4: (9, 256), 8: (4, 256)}
        assert num_ranks in table, f"Unsupported number of EP ranks: {num_ranks}"
        s, r = table[num_ranks]
        return _C().Config(Buffer.num_sms, s, r, 6, 128)

    def _is_internode(self) -> bool:
        return False

    def _blocks(self, config) -> int:
        if self._push_blocks:
            return self._push_blocks
        n = config.num_sms if config is not None else Buffer.num_sms
        return max(1, int(n))

    # ------------------------------------------------------------------ dispatch
    def _dispatch_begin(self, x, topk_idx, topk_weights, num_experts, tile_m, dispatch_seq, capacity_mode=False):
        if dispatch_seq is None:
            self._next_seq += 1
            seq = self._next_seq
        else:
            seq = int(dispatch_seq)
        if topk_idx.dtype != torch.int64:
            topk_idx = topk_idx.to(torch.int64)
        st = self.runtime.dispatch_begin(x.contiguous(), topk_idx.contiguous(),
                                         topk_weights.contiguous().float(), num_experts, tile_m, seq, bool(capacity_mode))
        return st, seq

    def _make_handle(self, st, is_token_in_rank, seq, tile_m) -> StreamingHandle:
        return StreamingHandle(
            pool=st.pool, pool_topk_weight=st.pool_topk_weight, pool_recv_token=st.pool_recv_token,
            pool_k_slot=st.pool_k_slot, send_head=st.send_head,
            is_token_in_rank=is_token_in_rank if is_token_in_rank is not None else st.is_token_in_rank,
            rank_prefix_matrix=st.rank_prefix_matrix, channel_prefix_matrix=st.channel_prefix_matrix,
            recv_channel_prefix_matrix=st.recv_channel_prefix_matrix,
            expert_frequency=st.expert_frequency, expert_pool_block_offset=st.expert_pool_block_offset,
            base_pool=st.base_pool, seen_per_substream=st.seen_per_substream,
            tile_id_to_expert=st.tile_id_to_expert, pool_arrival_target=st.pool_arrival_target,
            pool_arrival_count=st.pool_arrival_count, k_local_remaining=st.k_local_remaining,
            y_done_per_token=st.y_done_per_token, o=st.o, recv_token_to_slots=st.recv_token_to_slots,
            k_local_total=st.k_local_total, total_tiles=st.total_tiles, tile_m=tile_m,
            TK_padded=st.total_tiles * tile_m, dispatch_seq=seq, _dispatch_out=st)

    def dispatch(self, x: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor,
                 is_token_in_rank: Optional[torch.Tensor], num_experts: int, *,
                 expert_alignment: int = 1, tile_m: int = 128, dispatch_seq: Optional[int] = None,
                 config=None, launch_push: bool = True, capacity_mode: bool = False):
        """Pool-layout dispatch (reference: stream_ep/buffer.py:493-610).

        Two kernels and one host poll: the metadata kernel (count exchange +
        layout for every rank), a host read of ``total_tiles`` / ``T_recv`` to size
        the pool exactly, and the push kernel.  Runs on the current stream.
        Returns ``(pool, handle, metadata_done_event)``; the event is recorded
        before the push kernel so consumers can read metadata while rows are
        still arriving and gate per tile on ``pool_arrival_count``.

        ``launch_push=False`` stops before the push kernel (the fused
        dispatch+GEMM-A kernel of ``stream_moe`` ships the rows itself).

        ``capacity_mode=True`` (after :meth:`enable_capacity_mode`) receives into a fixed region without the
        host read: the handle's tensors then span the region's capacity (``total_tiles``, ``TK_padded`` and
        ``num_recv_tokens`` are capacities, tiles past the live count have target 0) and the live sizes are
        the device tensor ``handle._dispatch_out.dev_sizes``.
        """
        assert expert_alignment == 1, "expert_alignment other than 1 is not supported"
        st, seq = self._dispatch_begin(x, topk_idx, topk_weights, num_experts, tile_m, dispatch_seq, capacity_mode)
        cfg = self.get_dispatch_config(self.group_size) if config is None else config
        if not self._emulated:
            self.runtime.dispatch_metadata(st, 3)
            self._allocate(st)
            if launch_push:
                self.runtime.dispatch_push(st, 7, self._blocks(cfg))
        else:
            self.runtime.dispatch_metadata(st, 1)
            self._phase()
            self.runtime.dispatch_metadata(st, 2)
            self._allocate(st)
            if launch_push:
                self.runtime.dispatch_push(st, 1, 1)
                self._phase()
                self.runtime.dispatch_push(st, 2, self._blocks(cfg))
                self._phase()
                self.runtime.dispatch_push(st, 4, 8)
        handle = self._make_handle(st, is_token_in_rank, seq, tile_m)
        return st.pool, handle, st.metadata_done_event

    def _allocate(self, st) -> None:
        """Host poll for the receive sizes + allocation of everything peers write into."""
        try:
            self.runtime.dispatch_allocate(st)
        except RuntimeError as e:
            if "timed out" in str(e) or "metadata failed" in str(e):
                raise StreamEPTimeout(str(e)) from None
            raise

    # ------------------------------------------------------------------ dispatch_grads
    def dispatch_grads(self, handle: StreamingHandle, dL_dy: torch.Tensor, *,
                       dispatch_seq: Optional[int] = None, config=None, launch_push: bool = True,
                       fused_buffers: bool = False):
        """Backward dispatch along the forward routing (reference:
        stream_ep/buffer.py:613-667).  Returns ``(dL_do_pool,
        bwd_dispatch_arrival_count, grads_started_event)``."""
        st = handle._dispatch_out
        g = self.runtime.grads_begin(st, fused_buffers)
        if launch_push:
            cfg = self.get_dispatch_config(self.group_size) if config is None else config
            dL_dy = dL_dy.contiguous()
            if not self._emulated:
                self.runtime.grads_push(st, g, dL_dy, 7, self._blocks(cfg))
            else:
                self.runtime.grads_push(st, g, dL_dy, 1, 1)
                self._phase()
                self.runtime.grads_push(st, g, dL_dy, 2, self._blocks(cfg))
                self._phase()
                self.runtime.grads_push(st, g, dL_dy, 4, 8)
        handle._grads_state = g
        return g.dl_do_pool, g.bwd_dispatch_arrival_count, g.started_event

    # ------------------------------------------------------------------ combine
    def combine(self, x: torch.Tensor, handle: StreamingHandle, *, combine_seq: Optional[int] = None,
                config=None) -> Tuple[torch.Tensor, None]:
        """Reduce per-recv-token rows back to their source tokens (reference:
        stream_ep/buffer.py:670-722).  Each source rank waits, per token and per
        contributing rank, for ``handle.y_done_per_token[r] >= combine_seq`` in the
        owner's memory, then reads the row over NVLink and accumulates in fp32."""
        seq = handle.dispatch_seq if combine_seq is None else combine_seq
        st = handle._dispatch_out
        c = self.runtime.combine_begin(st, x, handle.y_done_per_token, None, True)
        cfg = self.get_combine_config(self.group_size) if config is None else config
        self._combine_launch(st, c, True, int(seq), cfg)
        return c.out, None

    def combine_grads(self, dL_dx_per_r: torch.Tensor, handle: StreamingHandle,
                      weight_grads: torch.Tensor, bwd_a_done_per_token: torch.Tensor, *,
                      dispatch_seq: Optional[int] = None, config=None):
        """Backward combine (reference: stream_ep/buffer.py:725-780): returns
        ``(dL_dx [T, H] bf16, dL_dtopk_weights [T, K] f32)``."""
        seq = handle.dispatch_seq if dispatch_seq is None else dispatch_seq
        st = handle._dispatch_out
        c = self.runtime.combine_begin(st, dL_dx_per_r, bwd_a_done_per_token, weight_grads, False)
        cfg = self.get_combine_config(self.group_size) if config is None else config
        self._combine_launch(st, c, False, int(seq), cfg)
        return c.out, c.out_topk_weights

    def _combine_launch(self, st, c, is_fwd, seq, cfg):
        if not self._emulated:
            self.runtime.combine_launch(st, c, is_fwd, seq, 7, self._blocks(cfg))
        else:
            self.runtime.combine_launch(st, c, is_fwd, seq, 1, 1)
            self._phase()
            self.runtime.combine_launch(st, c, is_fwd, seq, 2, self._blocks(cfg))
            self._phase()   # every rank's gather is enqueued before anyone reuses the rows it reads

    @property
    def _emulated(self) -> bool:
        return self._local is not None and self.group_size > 1

    def _phase(self) -> None:
        """Phase boundary of a collective: a thread barrier for emulated ranks, nothing otherwise."""
        if self._local is not None:
            self._local[0]._barrier_wait()

    def barrier(self) -> None:
        """Device-side barrier over the group on the current stream (bounded wait)."""
        if self._emulated:
            raise StreamEPError("the device barrier waits for its peers and cannot be emulated on one GPU")
        self.runtime.barrier()


class LocalWorld:
    """Several ranks emulated in ONE process on ONE device.

    Kernels of different ranks that wait on one another must never run as
    separate launches on one GPU, so every collective of an emulated rank is
    issued phase by phase on ONE shared stream: first the phase that only writes
    (count exchange, record publish, row push) for all ranks, then the phase that
    reads.  Each rank runs in its own Python thread and the threads meet at a
    barrier between phases, so no kernel ever waits for a kernel that has not
    been enqueued before it.  Used by the single-GPU tests of the multi-rank
    data paths; production runs one process per GPU.
    """

    def __init__(self, num_ranks: int, arena_bytes: int = 256 << 20, timeout_ms: int = 2000,
                 allocator: Optional[str] = None):
        import threading
        self.num_ranks = num_ranks
        self._barrier = threading.Barrier(num_ranks)
        self._in_run = threading.local()
        self._static_bases = [None] * num_ranks
        self.buffers: List[Buffer] = [
            Buffer(None, arena_bytes, _local=(self, r), timeout_ms=timeout_ms, allocator=allocator) for r in range(num_ranks)]
        ptrs = [b.runtime.get_local_base_ptr() for b in self.buffers]
        for b in self.buffers:
            b.runtime.sync_local(ptrs)

    def size(self):
        return self.num_ranks

    def make_streams(self):
        """Both layer streams are the device's default stream: emulated ranks share one queue."""
        from .stream_moe.stream_moe import StreamHolder
        s = torch.cuda.default_stream()
        return StreamHolder(communicate=s, compute=s)

    def _barrier_wait(self):
        if self.num_ranks == 1:
            return
        if not getattr(self._in_run, "active", False):
            raise StreamEPError("collectives of an emulated rank must be called through LocalWorld.run")
        self._barrier.wait(timeout=120)

    def run(self, fn):
        """Call ``fn(rank, buffer)`` for every rank, each in its own thread; returns the results."""
        import threading
        results = [None] * self.num_ranks
        errors = [None] * self.num_ranks
        dev = torch.cuda.current_device()

        def work(r):
            self._in_run.active = True
            try:
                torch.cuda.set_device(dev)
                results[r] = fn(r, self.buffers[r])
            except BaseException as e:  # noqa: BLE001
                errors[r] = e
                self._barrier.abort()
        if self.num_ranks == 1:
            self._in_run.active = True
            try:
                return [fn(0, self.buffers[0])]
            finally:
                self._in_run.active = False
        threads = [threading.Thread(target=work, args=(r,)) for r in range(self.num_ranks)]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        if any(e is not None for e in errors):
            self._barrier.reset()
            first = next(e for e in errors if e is not None and not isinstance(e, threading.BrokenBarrierError)) \
                if any(e is not None and not isinstance(e, threading.BrokenBarrierError) for e in errors) \
                else next(e for e in errors if e is not None)
            raise first
        return results

    def check_status(self):
        msgs = []
        for b in self.buffers:
            m = b.runtime.poll_status(True)
            if m:
                msgs.append(f"rank {b.rank}: {m}")
        if msgs:
            if all("capacity overflow" in m for m in msgs):
                raise StreamEPOverflow("; ".join(msgs))
            raise StreamEPTimeout("; ".join(msgs))

    def enable_capacity_mode(self, *args, **kwargs):
        for b in self.buffers:
            b.enable_capacity_mode(*args, **kwargs)

    # convenience wrappers used by the tests ------------------------------------------------------
    def dispatch(self, xs, topk_idxs, topk_weights, num_experts, tile_m=128, seqs=None):
        out = self.run(lambda r, b: b.dispatch(xs[r], topk_idxs[r], topk_weights[r], None, num_experts,
                                               tile_m=tile_m, dispatch_seq=None if seqs is None else seqs[r]))
        return [h for _, h, _ in out]

    def dispatch_grads(self, handles, dL_dys):
        out = self.run(lambda r, b: b.dispatch_grads(handles[r], dL_dys[r]))
        return [(p, c) for p, c, _ in out]

    def combine(self, xs, handles, seqs=None):
        out = self.run(lambda r, b: b.combine(xs[r], handles[r], combine_seq=None if seqs is None else seqs[r]))
        return [o for o, _ in out]

    def combine_grads(self, dxs, handles, weight_grads, dones, seqs=None):
        return self.run(lambda r, b: b.combine_grads(dxs[r], handles[r], weight_grads[r], dones[r],
                                                     dispatch_seq=None if seqs is None else seqs[r]))
