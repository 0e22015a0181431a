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


def _pointer_table(tensors):
    import ctypes

    return (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


def exchange_device_buffers(tensor, info: RankInfo, group=None):
    """Every rank's `tensor` (device memory from the ordinary allocator) as a tensor usable from this
    process: the list holds this rank's own tensor at `info.rank` and, for the others, mappings of
    their memory opened from the CUDA inter-process handles the ranks exchange through the process
    group.  The owner must keep its tensor alive as long as any peer uses the mapping."""
    if info.world == 1:
        return [tensor]
    from torch.multiprocessing.reductions import reduce_tensor

    rebuild, args = reduce_tensor(tensor)
    handles = [None] * info.world
    dist.all_gather_object(handles, (rebuild, args), group=group)
    peers = []
    for g, (fn, a) in enumerate(handles):
        peers.append(tensor if g == info.rank else fn(*a))
    for g, t in enumerate(peers):
        if g != info.rank and t.device != tensor.device:
            if not torch.cuda.can_device_access_peer(tensor.device.index, t.device.index):
                raise RuntimeError(f"GPU {tensor.device.index} cannot address the memory of GPU {t.device.index}")
            # a first copy between the two devices switches peer access on for this process
            torch.empty(1, dtype=t.dtype, device=tensor.device).copy_(t.reshape(-1)[:1])
    return peers


class FusedColumnParallelLinear(torch.nn.Module):
    """`ColumnParallelLinear` for the per-tensor FP8 linear with the exchange inside the GEMM.

    Every rank holds two full [max_rows, N] bf16 output buffers and maps all its peers' buffers.
    A call quantizes the (replicated) activations, runs ONE kernel that computes this rank's N / G
    columns and stores each finished chunk into the same place of every rank's buffer
    (`rk_gemm_fp8_column_parallel`), and then a one-warp kernel that waits until every peer's slab
    has arrived (`rk_wait_peers`): no collective launch, no gather copy, and the transfer of early
    tiles overlaps the computation of later ones.  The result is a view of an internal buffer and
    stays valid until the call after the next one (the two buffers alternate)."""

    def __init__(self, linear, info: RankInfo, max_rows, make_linear=None, group=None):
        super().__init__()
        from . import _lib

        n = linear.out_features
        if n % info.world or (n // info.world) % 8:
            raise ValueError(f"out_features {n} does not split into slabs of a multiple of 8 columns over {info.world} ranks")
        full = make_linear(linear) if make_linear is not None else linear
        if type(full).__name__ != "Fp8CutlassLinear" or full.mode != "per_tensor":
            raise TypeError("the fused exchange is built for the per-tensor FP8 linear")
        self.info, self.out_features, self.in_features = info, n, full.in_features
        self.slab = n // info.world
        self.local = shard_rows(full, info.rank * self.slab, (info.rank + 1) * self.slab)
        self.max_rows = int(max_rows)
        device = full.packed_weight.device
        self.device = device
        self.buffers = [torch.zeros((self.max_rows, n), dtype=torch.bfloat16, device=device) for _ in range(2)]
        self.flags = torch.zeros(max(info.world, 8), dtype=torch.int32, device=device)
        torch.cuda.synchronize(device)
        self._peer_buffers = [exchange_device_buffers(b, info, group) for b in self.buffers]  # keeps the mappings open
        self._peer_flags = exchange_device_buffers(self.flags, info, group)
        self._flag_table = _pointer_table(self._peer_flags)
        self._maps = {}  # rows -> the two descriptor arrays (one per output buffer)
        self.epoch = 0
        self._lib = _lib

    def _descriptors(self, rows):
        maps = self._maps.get(rows)
        if maps is None:
            L = self._lib
            maps = []
            for peers in self._peer_buffers:
                buf = torch.empty(128 * self.info.world, dtype=torch.uint8, device=self.device)
                code = L.load().rk_column_parallel_maps(_pointer_table(peers), self.info.world, rows, self.out_features,
                                                        self.info.rank * self.slab, self.slab, L.ptr(buf),
                                                        L.stream_ptr(self.device))
                L.check(code, "rk_column_parallel_maps")
                maps.append(buf)
            self._maps[rows] = maps
        return maps

    def forward(self, x):
        L = self._lib
        lead = x.shape[:-1]
        flat = x.reshape(-1, self.in_features)
        rows = flat.shape[0]
        if rows > self.max_rows:
            raise ValueError(f"{rows} rows exceed the {self.max_rows} rows the exchange buffers were sized for")
        # replicated activations: every rank derives the same per-tensor scale
        q, scale = self.local.pack_input(flat)
        self.epoch += 1
        which = self.epoch & 1
        maps = self._descriptors(rows)[which]
        with torch.cuda.device(self.device):
            ws = L.gemm_workspace(L.OP_FP8, self.device, rows, self.slab, self.in_features)
            stream = L.stream_ptr(self.device)
            code = L.load().rk_gemm_fp8_column_parallel(
                L.ptr(q), L.ptr(scale), L.ptr(self.local.packed_weight), L.ptr(self.local.weight_scale),
                L.ptr(self.local.bias), rows, self.slab, self.in_features, L.ptr(maps), self._flag_table, self.info.rank,
                self.info.world, self.epoch, L.ptr(ws), ws.numel(), stream)
            L.check(code, "rk_gemm_fp8_column_parallel")
            code = L.load().rk_wait_peers(L.ptr(self.flags), self.info.rank, self.info.world, self.epoch, L.ptr(ws),
                                          ws.numel(), stream)
            L.check(code, "rk_wait_peers")
        return self.buffers[which][:rows].view(*lead, self.out_features)
