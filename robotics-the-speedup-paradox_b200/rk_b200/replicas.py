"""Host-side helpers for running the quantized linears as independent replicas, one process per GPU.

The linears of independent environment rollouts never exchange data: every rank owns a full copy
of the packed weights and its own activations, so there is no data-path collective.  What the ranks
do share is measurement: a common start line (barrier) and the slowest rank's time (max over
ranks), from which whole-job throughput is the units all ranks processed divided by that time.
The same helpers run on CPU ranks (`gloo`) and GPU ranks (`nccl`).
"""

import os
import sys
from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class RankInfo:
    rank: int
    world: int
    local_rank: int


def rank_info(env=None) -> RankInfo:
    """Reads the launcher's RANK / WORLD_SIZE / LOCAL_RANK (defaults describe a single process)."""
    env = os.environ if env is None else env
    rank = int(env.get("RANK", "0"))
    world = int(env.get("WORLD_SIZE", "1"))
    local = int(env.get("LOCAL_RANK", "0"))
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"inconsistent launcher environment: RANK={rank} WORLD_SIZE={world}")
    return RankInfo(rank, world, local)


class _stdout_to_stderr:
    """Routes file descriptor 1 to stderr for a while: the communication library announces itself
    on stdout when its communicator is created, and stdout is reserved for the result line."""

    def __enter__(self):
        sys.stdout.flush()
        self.saved = os.dup(1)
        os.dup2(2, 1)
        return self

    def __exit__(self, *exc):
        sys.stdout.flush()
        os.dup2(self.saved, 1)
        os.close(self.saved)
        return False


def init(info: RankInfo, device: torch.device) -> None:
    """Joins the process group when there is more than one rank (nccl on GPUs, gloo on CPU) and runs
    one barrier so that the communicator exists before any timed region."""
    if info.world == 1 or dist.is_initialized():
        return
    with _stdout_to_stderr():
        if device.type == "cuda":
            dist.init_process_group("nccl", device_id=device)
            dist.barrier(device_ids=[device.index])
            torch.cuda.synchronize(device)
        else:
            dist.init_process_group("gloo")
            dist.barrier()


def barrier(info: RankInfo, device: torch.device) -> None:
    """All ranks arrive, and this rank's device is idle, before anyone continues."""
    if info.world > 1:
        if device.type == "cuda":
            dist.barrier(device_ids=[device.index])
        else:
            dist.barrier()
    if device.type == "cuda":
        torch.cuda.synchronize(device)


def max_over_ranks(values, info: RankInfo, device: torch.device):
    """Element-wise maximum of a short list of floats over all ranks (the slowest rank's times)."""
    t = torch.tensor(list(values), dtype=torch.float64, device=device)
    if info.world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.tolist()


def shard_range(total_units: int, info: RankInfo):
    """Contiguous slice [begin, end) of `total_units` independent units owned by this rank; the first
    `total_units % world` ranks take one extra unit.  Used when a fixed job is split (strong scaling)."""
    if total_units < 0:
        raise ValueError("total_units must be non-negative")
    base, extra = divmod(total_units, info.world)
    begin = info.rank * base + min(info.rank, extra)
    return begin, begin + base + (1 if info.rank < extra else 0)


def whole_job_rate(units_per_rank: float, info: RankInfo, slowest_ms: float) -> float:
    """Units per second of the whole job when every rank processed `units_per_rank` (weak scaling)."""
    if slowest_ms <= 0:
        raise ValueError("elapsed time must be positive")
    return units_per_rank * info.world / (slowest_ms * 1e-3)


def finish() -> None:
    if dist.is_initialized():
        dist.destroy_process_group()


def shard_rows(module, begin, end):
    """Rows [begin, end) of the output channels of a linear as a module of the same kind.

    A quantized linear is sliced AFTER quantization: the slab takes the matching rows of the packed
    codes and of the per-row scales (or 128-row scale-factor blocks) and SHARES the per-tensor
    scale of the whole weight, so that every slab computes exactly the columns the one-GPU linear
    computes.  (Quantizing each slab by itself would give every slab its own per-tensor scale and a
    slightly different result.)  Any module exposing `shard_output_rows(begin, end)` slices itself."""
    if hasattr(module, "shard_output_rows"):
        return module.shard_output_rows(begin, end)
    if isinstance(module, torch.nn.Linear):
        shard = torch.nn.Linear(module.in_features, end - begin, bias=module.bias is not None,
                                device=module.weight.device, dtype=module.weight.dtype)
        with torch.no_grad():
            shard.weight.copy_(module.weight[begin:end])
            if module.bias is not None:
                shard.bias.copy_(module.bias[begin:end])
        return shard.requires_grad_(False)
    kind = type(module).__name__
    bias = None if getattr(module, "bias", None) is None else module.bias[begin:end].contiguous()
    rows = end - begin
    if kind == "IntegerLinear":
        return type(module)(module.packed_weight[begin:end].contiguous(), module.weight_scale[begin:end].contiguous(),
                            bias, module.in_features, rows, module.bits, module.tactic, module.pack_reuse,
                            module.biasless_epilogue)
    if kind == "W4A16Linear":
        return type(module)(module.packed_weight[begin:end].contiguous(), module.weight_scale[:, begin:end].contiguous(),
                            bias, module.in_features, rows, module.tactic)
    if kind in ("Fp8CutlassLinear", "Fp4CutlassLinear"):
        codes = module.packed_weight[begin:end].contiguous()
        block_scaled = kind == "Fp4CutlassLinear" or module.mode == "mxfp8"
        scale = module.weight_scale  # per-tensor: one shared scalar
        if block_scaled:
            # scale factors live in 512-byte chunks per 128 rows: a slab is whole row blocks
            if begin % 128 or (rows % 128 and end != module.out_features):
                raise ValueError("block-scaled slabs must start and end on multiples of 128 rows")
            per_block = module.weight_scale.numel() // ((module.out_features + 127) // 128)
            scale = module.weight_scale[begin // 128 * per_block:(end + 127) // 128 * per_block].contiguous()
        if kind == "Fp8CutlassLinear":
            return type(module)(codes, scale, bias, module.in_features, rows, module.role, module.target_name, module.mode)
        return type(module)(codes, scale, module.weight_global_scale, bias, module.in_features, rows, module.role,
                            module.target_name)
    raise TypeError(f"do not know how to take output rows of a {kind}")


class ColumnParallelLinear(torch.nn.Module):
    """One exchange step across GPUs: the widest projections (gate/up, N = 16384) split along N.

    The full linear is quantized ONCE (`make_linear`, or it already is a quantized module); rank r
    then keeps rows [r * N / G, (r + 1) * N / G) of its packed codes and scales (`shard_rows`) and
    the shared per-tensor scale.  Activations are replicated; every rank computes its [M, N / G]
    slab and an all-gather assembles [M, N] on all ranks - bit-identical to the one-GPU output."""

    def __init__(self, linear, info: RankInfo, make_linear=None):
        super().__init__()
        n = linear.out_features
        if n % info.world:
            raise ValueError(f"out_features {n} does not split evenly over {info.world} ranks")
        self.info = info
        self.out_features = n
        self.in_features = linear.in_features
        self.slab = n // info.world
        full = make_linear(linear) if make_linear is not None else linear
        self.local = shard_rows(full, info.rank * self.slab, (info.rank + 1) * self.slab)

    def forward(self, x):
        part = self.local(x)  # [..., N / G]
        if self.info.world == 1:
            return part
        lead = part.shape[:-1]
        flat = part.reshape(-1, self.slab).contiguous()
        rows = flat.shape[0]
        gathered = torch.empty((self.info.world * rows, self.slab), device=flat.device, dtype=flat.dtype)
        dist.all_gather_into_tensor(gathered, flat)  # rank r's slab lands in rows [r * M, (r + 1) * M)
        # [G, M, N / G] -> [M, G * N / G]: rank order along N is the order of the weight rows
        return gathered.view(self.info.world, rows, self.slab).permute(1, 0, 2).reshape(*lead, self.out_features)


class _DevicePointer:
    """Lets torch view device memory that this module owns (`torch.as_tensor` reads the interface)."""

    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class ExchangeMemory:
    """One block of device memory per rank that every other rank of the node maps.

    `rk_peer_alloc` allocates the block and returns its inter-process handle; the handles travel
    through the process group; `rk_peer_open` maps every peer's block with THIS rank's device
    current, which is what makes the mapping usable by kernels running here.  `pointers[g]` is
    rank g's block as seen from this process (this rank's own allocation at `info.rank`)."""

    def __init__(self, nbytes, device, info: RankInfo, group=None):
        import ctypes

        from . import _lib

        self._lib, self.info, self.device, self.nbytes = _lib, info, device, int(nbytes)
        self._opened, self._group = [], group
        lib = _lib.load()
        ptr, handle = ctypes.c_void_p(), (ctypes.c_ubyte * 64)()
        with torch.cuda.device(device):
            _lib.check(lib.rk_peer_alloc(self.nbytes, ctypes.byref(ptr), handle), "rk_peer_alloc")
        self.ptr = ptr.value
        self.pointers = [self.ptr]
        if info.world > 1:
            gathered = [None] * info.world
            dist.all_gather_object(gathered, (bytes(handle), device.index), group=group)
            self.pointers = []
            with torch.cuda.device(device):
                for g, (peer_handle, owner) in enumerate(gathered):
                    if g == info.rank:
                        self.pointers.append(self.ptr)
                        continue
                    mapped = ctypes.c_void_p()
                    buf = (ctypes.c_ubyte * 64).from_buffer_copy(peer_handle)
                    _lib.check(lib.rk_peer_open(buf, owner, ctypes.byref(mapped)), "rk_peer_open")
                    self._opened.append(mapped.value)
                    self.pointers.append(mapped.value)
        self._view = torch.as_tensor(_DevicePointer(self.ptr, self.nbytes), device=device)

    def tensor(self, offset, shape, dtype):
        """A tensor over [offset, offset + size) of this rank's own block."""
        count = 1
        for d in shape:
            count *= d
        nbytes = count * torch.empty(0, dtype=dtype).element_size()
        return self._view[offset:offset + nbytes].view(dtype).view(*shape)

    def close(self):
        """Unmaps the peers' blocks, waits until every rank has done so, and frees this rank's block
        (an allocation must not be freed while another process still maps it).  Collective: every
        rank calls it, after all of them have stopped using the memory."""
        lib = self._lib.load()
        with torch.cuda.device(self.device):
            torch.cuda.synchronize(self.device)
            for p in self._opened:
                lib.rk_peer_close(p)
            self._opened = []
            if self.info.world > 1 and dist.is_initialized():
                dist.barrier(group=self._group, device_ids=[self.device.index])
            if self.ptr:
                self._view = None
                lib.rk_peer_free(self.ptr)
                self.ptr = 0


class SymmetricExchangeMemory:
    """The same block per rank as `ExchangeMemory`, from torch's symmetric-memory allocator, which also
    binds the ranks' blocks to one NVSwitch multicast object: `multicast_ptr` is an address whose
    stores (`multimem.st`) the switch delivers to every rank's block.  `pointers[g]` are the plain
    peer mappings.  Raises when the allocator, the rendezvous or the multicast binding is missing."""

    def __init__(self, nbytes, device, info: RankInfo, group=None):
        import torch.distributed._symmetric_memory as symm

        self.info, self.device, self.nbytes = info, device, int(nbytes)
        group = group if group is not None else dist.group.WORLD
        with torch.cuda.device(device):
            self._view = symm.empty((self.nbytes,), dtype=torch.uint8, device=device)
            self._handle = symm.rendezvous(self._view, group.group_name)
            self._view.zero_()
            torch.cuda.synchronize(device)
        self.pointers = [int(p) for p in self._handle.buffer_ptrs]
        self.multicast_ptr = int(getattr(self._handle, "multicast_ptr", 0) or 0)
        self.ptr = self.pointers[info.rank]
        if self.multicast_ptr == 0:
            raise RuntimeError("no multicast object behind the symmetric memory of this group")
        dist.barrier(group=group, device_ids=[device.index])  # every block is zero before anyone stores into it

    tensor = ExchangeMemory.tensor

    def close(self):
        torch.cuda.synchronize(self.device)
        self._view, self._handle = None, None


def _pointer_array(values):
    import ctypes

    return (ctypes.c_void_p * len(values))(*values)


def _all_ranks_agree(ok, info: RankInfo, group=None):
    if info.world == 1:
        return ok
    votes = [None] * info.world
    dist.all_gather_object(votes, bool(ok), group=group)
    return all(votes)


class FusedColumnParallelLinear(torch.nn.Module):
    """`ColumnParallelLinear` for the per-tensor FP8 linear with the exchange inside the GEMM.

    Every rank holds two full [max_rows, N] bf16 output buffers and maps all its peers' buffers.
    A call quantizes the (replicated) activations, runs ONE kernel that computes this rank's N / G
    columns and stores each finished chunk into the same place of every rank's buffer
    (`rk_gemm_fp8_column_parallel`), and then a one-warp kernel that waits until every peer's slab
    has arrived (`rk_wait_peers`): no collective launch, no gather copy, and the transfer of early
    tiles overlaps the computation of later ones.

    `transport`: "peer" (the default) - CUDA inter-process mappings and one TMA store per
    destination: the rank's own copy stays on its GPU and (G - 1) / G of the output crosses the
    links in each direction; "multicast" - the buffers come from torch's symmetric memory and the
    kernel stores to their NVSwitch multicast address: one copy of the slab leaves each GPU, but
    every GPU then RECEIVES the whole output over its links, its own slab included.  An all-gather
    is bound by what each GPU receives, so multicast does not help it (measured slower on two GPUs).

    The result is a view of an internal buffer and stays valid until the call after the next one
    (the two buffers alternate).  Every rank must make the same sequence of calls; `close()` (after
    a barrier of the ranks) releases the memory.  The call counter that the ranks compare lives in
    device memory, so the calls may be captured in a CUDA graph - with an even number of calls per
    graph, because the buffer a call writes is fixed at capture."""

    def __init__(self, linear, info: RankInfo, max_rows, make_linear=None, group=None, transport=None):
        super().__init__()
        from . import _lib

        n = linear.out_features
        if n % info.world or (n // info.world) % 8:
            raise ValueError(f"out_features {n} does not split into slabs of a multiple of 8 columns over {info.world} ranks")
        if transport not in (None, "multicast", "peer"):
            raise ValueError("transport must be 'peer' (also None) or 'multicast'")
        full = make_linear(linear) if make_linear is not None else linear
        if type(full).__name__ != "Fp8CutlassLinear" or full.mode != "per_tensor":
            raise TypeError("the fused exchange is built for the per-tensor FP8 linear")
        self.info, self.out_features, self.in_features = info, n, full.in_features
        self.slab = n // info.world
        self.local = shard_rows(full, info.rank * self.slab, (info.rank + 1) * self.slab)
        self.max_rows = int(max_rows)
        device = full.packed_weight.device
        self.device = device
        # one block: two output buffers, then the flag array and this rank's call counter
        self._buffer_bytes = (self.max_rows * n * 2 + 255) // 256 * 256
        nbytes = 2 * self._buffer_bytes + 256
        self.memory, self.transport, self.multicast_error = None, "peer", None
        if transport == "multicast" and info.world > 1:
            memory = None
            try:
                memory = SymmetricExchangeMemory(nbytes, device, info, group)
            except Exception as exc:  # reported; the peer transport takes over unless multicast was demanded
                self.multicast_error = f"{type(exc).__name__}: {exc}"
            if _all_ranks_agree(memory is not None, info, group):
                self.memory, self.transport = memory, "multicast"
            elif transport == "multicast":
                raise RuntimeError(f"multicast transport unavailable: {self.multicast_error or 'another rank failed'}")
        if self.memory is None:
            self.memory = ExchangeMemory(nbytes, device, info, group)
        self.buffers = [self.memory.tensor(i * self._buffer_bytes, (self.max_rows, n), torch.bfloat16) for i in range(2)]
        self.flags = self.memory.tensor(2 * self._buffer_bytes, (8,), torch.int32)
        self.epoch_counter = self.memory.tensor(2 * self._buffer_bytes + 64, (1,), torch.int32)  # this rank's calls, on the device
        self.wait_counter = self.memory.tensor(2 * self._buffer_bytes + 128, (1,), torch.int32)  # the wait kernel's own count
        self._flag_table = _pointer_array([p + 2 * self._buffer_bytes for p in self.memory.pointers])
        self._out_tables = [_pointer_array([p + which * self._buffer_bytes for p in self.memory.pointers]) for which in range(2)]
        self.calls = 0  # host mirror: only its parity (which buffer) matters
        self._lib = _lib

    def forward(self, x):
        lead = x.shape[:-1]
        flat = x.reshape(-1, self.in_features)
        if flat.shape[0] > self.max_rows:
            raise ValueError(f"{flat.shape[0]} rows exceed the {self.max_rows} rows the exchange buffers were sized for")
        # replicated activations: every rank derives the same per-tensor scale
        q, scale = self.local.pack_input(flat)
        return self.forward_packed(q, scale).view(*lead, self.out_features)

    def forward_packed(self, q, scale):
        """e4m3 activations [rows, K] and their scale (the same on every rank) -> [rows, N] on every rank."""
        L = self._lib
        rows = q.shape[0]
        if rows > self.max_rows:
            raise ValueError(f"{rows} rows exceed the {self.max_rows} rows the exchange buffers were sized for")
        self.calls += 1
        which = self.calls & 1
        outs, multicast = None, None
        if self.transport == "multicast":
            multicast = self.memory.multicast_ptr + which * self._buffer_bytes
        else:
            outs = self._out_tables[which]
        with torch.cuda.device(self.device):
            ws = L.gemm_workspace(L.OP_FP8, self.device, rows, self.slab, self.in_features)
            stream = L.stream_ptr(self.device)
            code = L.load().rk_gemm_fp8_column_parallel(
                L.ptr(q), L.ptr(scale), L.ptr(self.local.packed_weight), L.ptr(self.local.weight_scale),
                L.ptr(self.local.bias), rows, self.slab, self.in_features, outs, multicast, self.out_features,
                self.info.rank * self.slab, self._flag_table, self.info.rank, self.info.world, L.ptr(self.epoch_counter),
                L.ptr(ws), ws.numel(), stream)
            L.check(code, "rk_gemm_fp8_column_parallel")
            code = L.load().rk_wait_peers(L.ptr(self.flags), self.info.world, L.ptr(self.wait_counter), L.ptr(ws), ws.numel(), stream)
            L.check(code, "rk_wait_peers")
        return self.buffers[which][:rows]

    def close(self):
        self.buffers, self.flags, self.epoch_counter, self.wait_counter = [], None, None, None
        self.memory.close()
