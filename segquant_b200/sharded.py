"""Column-sharded SegmentLinear: output features split over the ranks of a torch.distributed
process group (one process per GPU), activations replicated, one all-gather of output slices.

The reference has no distributed code at all; this is the multi-GPU form of its layer asked for by
the large-N GEMM sweep.  Rank r owns rows [r*N/g, (r+1)*N/g) of the weight (with their scales and
bias), quantises its own copy of x (cheaper than broadcasting the quantised bytes), runs the fused
layer forward on its slice and the slices are exchanged with NCCL `all_gather_into_tensor` over
NVLink.  The exchange moves (g-1)/g * M*N*2 bytes in and out of every GPU, which at B200 tensor
rates costs more than the GEMM itself for every K <= 12288; `forward` therefore reports nothing
by itself -- bench.py times the GEMM phase and the whole step separately.

forward_fused() is the fused form: the peers' output buffers are mapped into every process (symmetric
memory) and the GEMM epilogue stores each finished tile into all of them, so the exchange overlaps the
mainloop tile by tile and no gather kernel or interleave copy runs; only a barrier follows.
"""
import torch
import torch.distributed as dist


def shard_range(n_total, world, rank):
    """[begin, end) of the output columns rank `rank` owns; requires world | n_total so that all
    slices have one size and the gather is a single dense buffer."""
    if n_total % world:
        raise ValueError(f"N={n_total} is not divisible by world size {world}")
    per = n_total // world
    return rank * per, (rank + 1) * per


def assemble(gathered):
    """(world, M, N/world) rank-major gather buffer -> (M, N) with rank r's columns at
    [r*N/world, (r+1)*N/world)."""
    world, m, per = gathered.shape
    return gathered.permute(1, 0, 2).reshape(m, world * per)


def all_gather_slices(local, group=None):
    """All-gather equally shaped [M, N/world] slices into a (world, M, N/world) buffer."""
    world = dist.get_world_size(group)
    out = torch.empty((world,) + tuple(local.shape), dtype=local.dtype, device=local.device)
    local = local.contiguous()
    if dist.get_backend(group) == "nccl":
        dist.all_gather_into_tensor(out, local, group=group)
    else:
        dist.all_gather(list(out.unbind(0)), local, group=group)
    return out


class ColumnShardedSegLinear:
    """Holds this rank's slice as an ordinary SegmentLinear (real-quant)."""

    def __init__(self, local_layer, rank, world, n_total, group=None):
        self.layer, self.rank, self.world, self.n_total, self.group = local_layer, rank, world, n_total, group

    @classmethod
    def from_full(cls, x_calib, weight, bias, rank, world, kernel_type="Wint8Aint8", dual_scale=False, seg_mode="input",
                  chunks=1, chunksizes=None, weight_axis=1, group_size=None, group=None):
        from .layers.SegmentLinear import SegmentLinear
        n_total, k = weight.shape
        lo, hi = shard_range(n_total, world, rank)
        w_type, a_type = kernel_type[1:].split("A")
        w_args = {"real_quant": True, "axis": weight_axis}
        if group_size:
            w_args["group_size"] = group_size
        layer = SegmentLinear(k, hi - lo, bias=bias is not None, seg_mode=seg_mode, chunks=chunks, chunksizes=chunksizes,
                              custom_weight_tensor=weight[lo:hi].contiguous(),
                              custom_bias_tensor=None if bias is None else bias[lo:hi].contiguous(),
                              input_quant_type=a_type, weight_quant_type=w_type,
                              input_quant_args={"real_quant": True, "axis": None, "dual_scale": dual_scale},
                              weight_quant_args=w_args, device=weight.device)
        layer.calibrate(x_calib)
        layer.finish_calibrate()
        return cls(layer, rank, world, n_total, group)

    def local_forward(self, x):
        return self.layer(x)

    def forward(self, x):
        y = self.local_forward(x)
        lead = y.shape[:-1]
        gathered = all_gather_slices(y.reshape(-1, y.shape[-1]), self.group)
        return assemble(gathered).reshape(*lead, self.n_total)

    __call__ = forward

    # ---- fused all-gather: the GEMM epilogue stores every tile into all ranks' [M, N] buffers ----------
    def enable_fused_gather(self, max_rows, dtype=torch.bfloat16):
        """Allocate this rank's [max_rows, N] output in symmetric memory and exchange the mappings (one
        rendezvous; NCCL group).  After this, forward_fused() replaces local GEMM + all-gather + interleave."""
        import torch.distributed._symmetric_memory as symm
        dev = self.layer.bias_data.device if self.layer.bias_data is not None else self.layer.optimizer.weight_manager.device()
        group = self.group if self.group is not None else dist.group.WORLD
        self._full = symm.empty((max_rows, self.n_total), dtype=dtype, device=dev)
        self._handle = symm.rendezvous(self._full, group)
        self._peer_ptrs = [int(p) for r, p in enumerate(self._handle.buffer_ptrs) if r != self.rank]
        self._flag = torch.zeros(1, dtype=torch.int32, device=dev)

    def forward_fused(self, x):
        """x [M, K] (same on every rank).  Every rank's epilogue writes its column slice into its own buffer
        (TMA stores) and into every peer's buffer (plain stores over NVLink); a one-word all-reduce then orders all
        ranks' kernels before anyone reads.  Returns this rank's full [M, N] result (a view of the symmetric buffer:
        it is overwritten by the next call)."""
        m = x.shape[0]
        lo, hi = shard_range(self.n_total, self.world, self.rank)
        full = self._full[:m]
        self.layer(x.unsqueeze(0), out=full[:, lo:hi].unsqueeze(0), peer_outputs=(self._peer_ptrs, self.n_total, lo))
        dist.all_reduce(self._flag, group=self.group)   # stream-ordered barrier: completes after every rank's GEMM
        return full

    # bytes one GPU sends to its peers above which the NCCL all-gather is faster than the fused stores (measured on
    # 2 and 8 B200s: the epilogue's 32-row x 16-column boxes are 32-byte row segments on NVLink, which costs bandwidth
    # once the exchange, not the GEMM, sets the time)
    FUSED_MAX_BYTES = 70 * 1024 * 1024

    def forward_auto(self, x):
        """Fused exchange for small and medium outputs, NCCL all-gather for large ones.  x [M, K]."""
        out_bytes = x.shape[0] * (self.n_total // self.world) * 2 * (self.world - 1)
        if getattr(self, "_full", None) is not None and x.dim() == 2 and x.shape[0] <= self._full.shape[0] \
                and out_bytes <= self.FUSED_MAX_BYTES:
            return self.forward_fused(x)
        return self.forward(x)
