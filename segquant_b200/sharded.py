"""Column-sharded SegmentLinear: output features split over the ranks of a torch.distributed
process group (one process per GPU), activations replicated, one exchange of output column blocks.

The reference has no distributed code at all; this is the multi-GPU form of its layer asked for by
the large-N GEMM sweep.  Rank r owns rows [r*N/g, (r+1)*N/g) of the weight (with their scales and
bias), quantises its own copy of x (cheaper than broadcasting the quantised bytes: quantising reads
3 bytes per element from HBM, receiving them would move 1 byte per element over NVLink, which is an
order of magnitude slower) and runs the fused layer forward on its slice.  Three ways to exchange:

forward()        the baseline: NCCL `all_gather_into_tensor` of the [M, N/g] slices into a (g, M, N/g) buffer, then
                 a permuting copy into [M, N].
forward_push()   every rank's [M, N] result lives in symmetric memory; the GEMM writes the rank's column block in
                 place, then ONE kernel (ops.push_columns) stores that block into the same columns of every peer's
                 matrix: final layout, whole 512-byte row segments on the wire, no gather buffer, no permute.
forward_fused()  the exchange inside the GEMM epilogue: every finished tile goes to the rank's own matrix and to every
                 peer's by TMA stores ([32 rows x 128 bytes] boxes: whole 128-byte lines on NVLink) while the mainloop
                 of the next tiles runs, so the transfer overlaps the math tile by tile.
A barrier kernel on the compute stream (ops.peer_barrier: flag words in symmetric memory, a system-scope fence, a bounded
wait) orders the ranks after either of the last two.

Buffer rule of forward_push / forward_fused: results are views of TWO symmetric buffers used alternately.  The view
returned by call n is overwritten by PEERS during their call n + 2, which they can only start after this rank has
passed the barrier of call n + 1; so anything enqueued on the compute stream BEFORE this rank's call n + 1 may read
call n's result, and nothing later may.  (With a single buffer a peer's call n + 1 could overwrite the result while this
rank's consumers of call n were still running: the barrier after the GEMM only orders the GEMMs.)

The exchange moves (g-1)/g * M*N*2 bytes in and out of every GPU, which at B200 tensor rates costs more than the GEMM
itself for every K <= 12288 at g = 8; bench.py therefore reports GEMM-only, exchange and total times separately, next
to the NVLink-bound ceiling.
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


def row_range(m_total, world, rank):
    """[begin, end) of the input rows rank `rank` brings in from the host (forward_from_host_rows)."""
    per = (m_total + world - 1) // world
    return min(rank * per, m_total), min((rank + 1) * per, m_total)


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
        self._bufs, self._peer_ptrs, self._flags, self._flag_ptrs, self._epoch, self._calls = None, None, None, None, 0, 0

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

    def _device(self):
        opt = getattr(self.layer, "optimizer", None)
        return opt.weight_manager.device() if opt is not None else torch.device("cpu")

    def local_forward(self, x):
        return self.layer(x)

    def forward(self, x):
        y = self.local_forward(x)
        lead = y.shape[:-1]
        gathered = all_gather_slices(y.reshape(-1, y.shape[-1]), self.group)
        return assemble(gathered).reshape(*lead, self.n_total)

    __call__ = forward

    # ---- exchanges through symmetric memory --------------------------------------------------------------
    def enable_symmetric(self, max_rows, dtype=torch.bfloat16):
        """Allocate this rank's two [max_rows, N] result buffers in symmetric memory and exchange the mappings (one
        rendezvous each; NCCL group).  Needed once before forward_push() / forward_fused()."""
        import torch.distributed._symmetric_memory as symm
        dev = self._device()
        group = self.group if self.group is not None else dist.group.WORLD
        self._bufs, self._peer_ptrs = [], []
        for _ in range(2):
            buf = symm.empty((max_rows, self.n_total), dtype=dtype, device=dev)
            handle = symm.rendezvous(buf, group)
            self._bufs.append(buf)
            self._peer_ptrs.append([int(p) for r, p in enumerate(handle.buffer_ptrs) if r != self.rank])
        # barrier words: one array of `world` uint32 per rank, zero before anybody's first barrier
        flags = symm.empty((64,), dtype=torch.int32, device=dev)
        flags.zero_()
        torch.cuda.synchronize(dev)
        handle = symm.rendezvous(flags, group)
        self._flags, self._flag_ptrs = flags, [int(p) for p in handle.buffer_ptrs]
        dist.barrier(group=group)                      # every rank's words are zero before the first epoch is stored
        self._epoch = 0
        self._calls = 0

    enable_fused_gather = enable_symmetric      # earlier name

    def _next_buffer(self, m):
        if self._bufs is None:
            raise RuntimeError("call enable_symmetric(max_rows) first")
        if m > self._bufs[0].shape[0]:
            raise ValueError(f"{m} rows exceed the {self._bufs[0].shape[0]} rows the symmetric buffers were sized for")
        i = self._calls & 1
        self._calls += 1
        return self._bufs[i][:m], self._peer_ptrs[i]

    def _barrier(self):
        """Stream-ordered: completes on this rank once every rank has issued it, i.e. after every rank's stores into this
        rank's matrix have landed.  Epochs count the collective calls, the same on every rank."""
        from . import ops
        self._epoch += 1
        ops.peer_barrier(self.rank, self._flag_ptrs, self._epoch, self._device())

    def forward_push(self, x):
        """x [M, K] (same on every rank).  GEMM into this rank's columns of its own matrix, then one push of that block to
        every peer, then the barrier.  Returns this rank's full [M, N] result (see the buffer rule in the module docstring)."""
        from . import ops
        m = x.shape[0]
        lo, hi = shard_range(self.n_total, self.world, self.rank)
        full, peers = self._next_buffer(m)
        mine = full[:, lo:hi]
        self.layer(x.unsqueeze(0), out=mine.unsqueeze(0))
        esz = full.element_size()
        ops.push_columns(mine, [p + lo * esz for p in peers], self.n_total * esz)
        self._barrier()
        return full

    def forward_fused(self, x):
        """x [M, K] (same on every rank).  Every rank's epilogue writes its column block into its own matrix and into
        every peer's (TMA stores over NVLink) while the next tile's mainloop runs; then the barrier.  Returns this rank's
        full [M, N] result (see the buffer rule in the module docstring)."""
        m = x.shape[0]
        lo, hi = shard_range(self.n_total, self.world, self.rank)
        full, peers = self._next_buffer(m)
        self.layer(x.unsqueeze(0), out=full[:, lo:hi].unsqueeze(0), peer_outputs=(peers, self.n_total, lo))
        self._barrier()
        return full

    def forward_auto(self, x):
        """The fused exchange wherever the symmetric buffers allow it: measured the fastest of the three at 325 of 336
        points of the GEMM sweep on 2 GPUs and 138 of 144 on 4 (also where the exchange outlasts the GEMM several times
        over: the stores start as soon as the first tiles finish instead of after the last one); the NCCL all-gather
        otherwise.  x [M, K]."""
        if self._bufs is None or x.dim() != 2 or x.shape[0] > self._bufs[0].shape[0]:
            return self.forward(x)
        return self.forward_fused(x)

    def forward_from_host_rows(self, x_rows_host, m_total, exchange="auto"):
        """End-to-end form for inputs that start in HOST memory: every rank copies only ITS row block of x
        (row_range(m_total, world, rank), pinned memory) over PCIe, the blocks are all-gathered over NVLink into the
        replicated [M, K] activation (rows are contiguous, so the gather is the final layout), then the sharded forward
        runs.  The whole input crosses PCIe once in total instead of once per rank."""
        dev = self._device()
        k = x_rows_host.shape[1]
        lo, hi = row_range(m_total, self.world, self.rank)
        per = (m_total + self.world - 1) // self.world
        x_full = torch.empty((per * self.world, k), dtype=x_rows_host.dtype, device=dev)
        x_full[lo:hi].copy_(x_rows_host, non_blocking=True)
        if dist.get_backend(self.group) == "nccl":
            dist.all_gather_into_tensor(x_full, x_full[self.rank * per:(self.rank + 1) * per], group=self.group)
        else:
            parts = [torch.empty((per, k), dtype=x_full.dtype, device=dev) for _ in range(self.world)]
            dist.all_gather(parts, x_full[self.rank * per:(self.rank + 1) * per].contiguous(), group=self.group)
            x_full = torch.cat(parts)
        x = x_full[:m_total]
        fn = {"auto": self.forward_auto, "push": self.forward_push, "fused": self.forward_fused, "nccl": self.forward}[exchange]
        return fn(x)


class HostRowPipeline:
    """End-to-end driver of a column-sharded layer for inputs that live in HOST memory, one step in flight per stage.

    Per step every rank copies ITS row block of x from pinned host memory (copy stream), all-gathers the blocks over NVLink
    and runs the sharded forward (compute stream), and reads its row block of the result back into pinned host memory
    (read-back stream); consecutive steps overlap on the three streams, with two device input buffers used alternately.
    The rank's output rows are first copied to a private device buffer ON THE COMPUTE STREAM: the layer's symmetric result
    buffers may be overwritten by peers as soon as this rank has issued its next forward (see the module docstring), so
    nothing outside the compute stream may read them.  Without CUDA (gloo tests) the same steps run one after the other."""

    def __init__(self, layer, m_total, k, in_dtype, out_dtype, exchange="auto"):
        self.layer, self.m_total, self.exchange = layer, m_total, exchange
        dev = layer._device()
        self.dev, self.cuda = dev, dev.type == "cuda"
        w, r = layer.world, layer.rank
        self.per = (m_total + w - 1) // w
        self.lo, self.hi = row_range(m_total, w, r)
        self.x = [torch.empty((self.per * w, k), dtype=in_dtype, device=dev) for _ in range(2)]
        self.y_rows = [torch.empty((self.hi - self.lo, layer.n_total), dtype=out_dtype, device=dev) for _ in range(2)]
        if self.cuda:
            self.s_in, self.s_cmp, self.s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.Stream(dev)
            self.ev_in, self.ev_cmp, self.ev_out = ([torch.cuda.Event() for _ in range(2)] for _ in range(3))

    def _compute(self, b):
        lay = self.layer
        xf = self.x[b]
        mine = xf[lay.rank * self.per:(lay.rank + 1) * self.per]
        if dist.get_backend(lay.group) == "nccl":
            dist.all_gather_into_tensor(xf, mine, group=lay.group)
        else:
            parts = [torch.empty_like(mine) for _ in range(lay.world)]
            dist.all_gather(parts, mine.contiguous(), group=lay.group)
            xf.copy_(torch.cat(parts))
        fn = {"auto": lay.forward_auto, "push": lay.forward_push, "fused": lay.forward_fused, "nccl": lay.forward}[self.exchange]
        y = fn(xf[:self.m_total])
        self.y_rows[b].copy_(y[self.lo:self.hi])

    def step(self, i, x_rows_host, y_rows_host):
        """Enqueue step i: x_rows_host = this rank's rows of x (pinned), y_rows_host receives this rank's rows of y."""
        b = i & 1
        if not self.cuda:
            self.x[b][self.lo:self.hi].copy_(x_rows_host)
            self._compute(b)
            y_rows_host.copy_(self.y_rows[b])
            return
        with torch.cuda.stream(self.s_in):
            self.s_in.wait_event(self.ev_cmp[b])            # the forward two steps ago has consumed x[b]
            self.x[b][self.lo:self.hi].copy_(x_rows_host, non_blocking=True)
            self.ev_in[b].record(self.s_in)
        with torch.cuda.stream(self.s_cmp):
            self.s_cmp.wait_event(self.ev_in[b])
            self.s_cmp.wait_event(self.ev_out[b])           # y_rows[b] has been read back
            self._compute(b)
            self.ev_cmp[b].record(self.s_cmp)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(self.ev_cmp[b])
            y_rows_host.copy_(self.y_rows[b], non_blocking=True)
            self.ev_out[b].record(self.s_out)

    def run(self, n, x_rows_host, y_rows_host):
        """n steps from the two alternating pinned inputs x_rows_host[0 / 1]; returns after everything is enqueued and the
        caller's current stream has been made to wait for all three streams."""
        if self.cuda:
            cur = torch.cuda.current_stream(self.dev)
            for s in (self.s_in, self.s_cmp, self.s_out):
                s.wait_stream(cur)
        for i in range(n):
            self.step(i, x_rows_host[i & 1], y_rows_host)
        if self.cuda:
            for s in (self.s_in, self.s_cmp, self.s_out):
                cur.wait_stream(s)
