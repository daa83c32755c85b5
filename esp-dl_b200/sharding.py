"""Batch sharding across GPUs for the forward path: one process per GPU, a replica of the weights on each,
the images split into contiguous shards, and one exchange per step - the gather of the logits.

The path has no other cross-image dependency, so there is no collective between layers.  The helpers work on any
torch.distributed backend ("nccl" on GPUs, "gloo" in the CPU tests)."""
import torch
import torch.distributed as dist


def shard_range(total, rank, world):
    """[begin, end) of the images rank `rank` owns when `total` images are split over `world` ranks.
    Shards are contiguous and differ by at most one image; the first `total % world` ranks get the extra one."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    base, extra = divmod(total, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def gather_logits(local, total, group=None, out=None):
    """All ranks pass their shard's logits `local` [n_local, classes] (same dtype and device everywhere) and get the
    [total, classes] tensor of all images in image order.  Equal shards go through one all_gather_into_tensor on
    the caller's buffers; ragged shards are padded to the largest shard first."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    begin, end = shard_range(total, rank, world)
    if local.shape[0] != end - begin:
        raise ValueError(f"rank {rank} holds {local.shape[0]} rows, its shard has {end - begin}")
    classes = local.shape[1:]
    largest = shard_range(total, 0, world)[1]
    if total % world == 0:
        if out is None:
            out = torch.empty((total,) + tuple(classes), dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(out, local.contiguous(), group=group)
        return out
    padded = torch.zeros((largest,) + tuple(classes), dtype=local.dtype, device=local.device)
    padded[: local.shape[0]] = local
    pieces = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(pieces, padded, group=group)
    rows = [pieces[r][: shard_range(total, r, world)[1] - shard_range(total, r, world)[0]] for r in range(world)]
    return torch.cat(rows, dim=0)


# ---------------------------------------------------------------------------------------------------------------
# N-sharded Gemm: the filter [N][K] is split along N into one block of rows per rank, every rank holds all of the
# input [M][K] and computes out[:, n0:n1]; one all-gather along N assembles the [M][N] result on every rank.  K is
# not split, so no int32 partial sum ever crosses a GPU and every output is rounded exactly as on one GPU.
# (Gemm = conv2d on a {1,1,M,K} input with a {1,1,K,N} filter: esp-dl/dl/module/include/dl_module_gemm.hpp:85-123.)
# ---------------------------------------------------------------------------------------------------------------

def _interleave_columns(staging, out):
    """out[m, r*n_loc + j] = staging[r, m, j].  On a GPU this is one launch of the library's strided-copy kernel
    (espdl_b200_copy); host tensors (the gloo tests) are re-ordered by torch."""
    world, m, n_loc = staging.shape
    if not staging.is_cuda:
        out.copy_(staging.permute(1, 0, 2).reshape(m, world * n_loc))
        return out
    import ctypes as C
    from . import abi
    d = abi.CopyDesc()
    d.src, d.dst, d.elem_size, d.ndim = staging.data_ptr(), out.data_ptr(), staging.element_size(), 3
    for i, (s, a, b) in enumerate(zip((world, m, n_loc), (m * n_loc, n_loc, 1), (n_loc, world * n_loc, 1))):
        d.shape[i], d.src_stride[i], d.dst_stride[i] = s, a, b
    stream = C.c_void_p(torch.cuda.current_stream(staging.device).cuda_stream)
    abi.check(abi.load().espdl_b200_copy(C.byref(d), stream), "espdl_b200_copy")
    return out


def gather_columns(local, group=None, staging=None, out=None):
    """Every rank passes its [M, N/world] block of output columns and gets the whole [M, N] matrix: one
    all_gather_into_tensor into a [world, M, N/world] staging buffer, then a local re-ordering copy."""
    world = dist.get_world_size(group)
    m, n_loc = local.shape
    if staging is None:
        staging = torch.empty((world, m, n_loc), dtype=local.dtype, device=local.device)
    if out is None:
        out = torch.empty((m, world * n_loc), dtype=local.dtype, device=local.device)
    # collectives move bytes: NCCL has no 16-bit integer type
    dist.all_gather_into_tensor(staging.view(world * m, n_loc).view(torch.uint8), local.contiguous().view(torch.uint8),
                                group=group)
    return _interleave_columns(staging, out)


class NShardedGemm:
    """out[M][N] = requantise(in[M][K] . filter[N][K]^T + bias) with the filter rows split over the ranks of `group`.

    filter: numpy int8/int16 [N][K] (the reference's generic-C order), bias: int32/int64 [N] or None,
    filter_exponents: int (per tensor) or int array [N] (per channel).  N must be a multiple of the world size.
    Every rank passes the same arrays and keeps only its block of rows on its GPU.  forward() takes the whole input
    as a device tensor [M][K] and returns the whole output on every rank."""

    def __init__(self, filter, bias, in_exponent, filter_exponents, out_exponent, activation=0, round_mode=0,
                 group=None, device=None, mode="gather"):
        """mode "gather": every rank computes its block, one all-gather and an interleaving copy assemble [M][N].
        mode "peer" (int8, one machine): every rank's kernel stores its columns straight into the [M][N] result of
        all ranks through peer-mapped pointers (espdl_b200_gemm_scatter); a one-element all-reduce on the stream then
        orders every rank's reads behind every rank's kernel.  No gather, no copy.

        Peer mode returns a view of a library-owned buffer that OTHER GPUs write.  Two buffers per M are used in turn:
        the result of call i stays valid until call i+2 is enqueued, provided it is read on the stream forward() was
        called on (a rank's kernel of call i+2 starts only after the exchange of call i+1 has completed, which every
        rank enqueues behind its own readers of result i).  A caller that reads a result on another stream, or keeps
        it beyond the next call, has to copy it first."""
        import numpy as np
        from . import abi
        self.abi, self.lib, self.group = abi, abi.load(), group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        n, self.k = filter.shape
        if n % self.world:
            raise ValueError(f"N={n} is not a multiple of the {self.world} ranks")
        self.n, self.n_loc = n, n // self.world
        n0, n1 = self.rank * self.n_loc, (self.rank + 1) * self.n_loc
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        up = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(self.device)
        self.dtype = {np.dtype(np.int8): abi.DTYPE_INT8, np.dtype(np.int16): abi.DTYPE_INT16}[filter.dtype]
        self.torch_dtype = torch.int8 if filter.dtype == np.int8 else torch.int16
        self.filter = up(filter[n0:n1])
        self.bias = None if bias is None else up(bias[n0:n1])
        self.per_channel = int(np.ndim(filter_exponents) > 0)
        self.ew = up(np.asarray(filter_exponents, dtype=np.int32)[n0:n1]) if self.per_channel else None
        self.e_w = 0 if self.per_channel else int(filter_exponents)
        self.e_in, self.e_out, self.activation, self.round_mode = in_exponent, out_exponent, activation, round_mode
        self._bufs = {}
        if mode not in ("gather", "peer") or (mode == "peer" and self.dtype != abi.DTYPE_INT8):
            raise ValueError("mode is 'gather' or 'peer'; 'peer' takes int8 only")
        self.mode = mode
        self._peer = {}   # M -> two sets of (own buffer, peers' mapped buffers, tensor view), used in turn
        self._turn = {}   # M -> which set the next call writes
        self._flag = None

    def forward(self, x):
        import ctypes as C
        m, k = x.shape
        if k != self.k or x.dtype != self.torch_dtype or not x.is_cuda or not x.is_contiguous():
            raise ValueError("input must be a contiguous device tensor [M][K] of the filter's type")
        if self.mode == "peer":
            return self._forward_peer(x)
        if m not in self._bufs:
            self._bufs[m] = (torch.empty((self.world, m, self.n_loc), dtype=self.torch_dtype, device=self.device),
                             torch.empty((m, self.n), dtype=self.torch_dtype, device=self.device))
        staging, out = self._bufs[m]
        local = staging[self.rank]
        d = self.abi.ConvDesc()
        d.input, d.filter, d.output = x.data_ptr(), self.filter.data_ptr(), local.data_ptr()
        d.bias = None if self.bias is None else self.bias.data_ptr()
        d.filter_exponents = None if self.ew is None else self.ew.data_ptr()
        d.dtype, d.n, d.in_h, d.in_w, d.in_c = self.dtype, 1, 1, m, k
        d.out_h, d.out_w, d.out_c, d.kh, d.kw = 1, m, self.n_loc, 1, 1
        d.stride_h = d.stride_w = d.dilation_h = d.dilation_w = d.group = 1
        d.in_exponent, d.out_exponent, d.filter_exponent = self.e_in, self.e_out, self.e_w
        d.per_channel, d.activation, d.round_mode = self.per_channel, self.activation, self.round_mode
        stream = C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        self.abi.check(self.lib.espdl_b200_conv2d(C.byref(d), stream), "espdl_b200_conv2d")
        dist.all_gather_into_tensor(staging.view(self.world * m, self.n_loc).view(torch.uint8), local.view(torch.uint8),
                                    group=self.group)
        return _interleave_columns(staging, out)

    # ------------------------------------------------------------------------------------------------ peer stores
    class _DeviceArray:
        """A device buffer of the library seen by torch without a copy (the CUDA array interface)."""

        def __init__(self, ptr, shape, typestr):
            self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (int(ptr), False), "version": 2}

    def _peer_buffers(self, m):
        import ctypes as C
        if m in self._peer:
            self._turn[m] ^= 1
            return self._peer[m][self._turn[m]]
        self._peer[m] = [self._new_peer_set(m), self._new_peer_set(m)]
        self._turn[m] = 0
        return self._peer[m][0]

    def _new_peer_set(self, m):
        import ctypes as C
        own = C.c_void_p()
        self.abi.check(self.lib.espdl_b200_arena_alloc(m * self.n, C.byref(own)), "arena_alloc")
        handle = (C.c_ubyte * 64)()
        self.abi.check(self.lib.espdl_b200_ipc_export(own, handle), "ipc_export")
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle), group=self.group)
        peers = []
        for r, h in enumerate(handles):
            if r == self.rank:
                continue
            mapped = C.c_void_p()
            buf = (C.c_ubyte * 64).from_buffer_copy(h)
            self.abi.check(self.lib.espdl_b200_ipc_open(buf, C.byref(mapped)), "ipc_open")
            peers.append(mapped)
        view = torch.as_tensor(self._DeviceArray(own.value, (m, self.n), "|i1"), device=self.device)
        return (own, peers, view)

    def _forward_peer(self, x):
        import ctypes as C
        m = x.shape[0]
        own, peers, view = self._peer_buffers(m)
        n0 = self.rank * self.n_loc
        d = self.abi.ConvDesc()
        d.input, d.filter, d.output = x.data_ptr(), self.filter.data_ptr(), own.value + n0
        d.bias = None if self.bias is None else self.bias.data_ptr()
        d.filter_exponents = None if self.ew is None else self.ew.data_ptr()
        d.dtype, d.n, d.in_h, d.in_w, d.in_c = self.dtype, 1, 1, m, self.k
        d.out_h, d.out_w, d.out_c, d.kh, d.kw = 1, m, self.n_loc, 1, 1
        d.stride_h = d.stride_w = d.dilation_h = d.dilation_w = d.group = 1
        d.out_pixel_stride = self.n
        d.in_exponent, d.out_exponent, d.filter_exponent = self.e_in, self.e_out, self.e_w
        d.per_channel, d.activation, d.round_mode = self.per_channel, self.activation, self.round_mode
        targets = (C.c_void_p * max(len(peers), 1))(*[C.c_void_p(p.value + n0) for p in peers])
        stream = C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        self.abi.check(self.lib.espdl_b200_gemm_scatter(C.byref(d), targets, len(peers), stream), "espdl_b200_gemm_scatter")
        if self.world > 1:
            # stream-ordered exchange: it completes on a rank only after every rank's kernel before it has completed
            if self._flag is None:
                self._flag = torch.zeros(1, dtype=torch.int32, device=self.device)
            dist.all_reduce(self._flag, group=self.group)
        return view

    def close(self):
        """Unmaps the peers' buffers and frees the own ones; every rank calls it (it synchronises the ranks first)."""
        if not self._peer:
            return
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier(group=self.group)
        sets = [s for pair in self._peer.values() for s in pair]
        for own, peers, _ in sets:
            for p in peers:
                self.lib.espdl_b200_ipc_close(p)
        if self.world > 1:
            dist.barrier(group=self.group)
        for own, _, _ in sets:
            self.lib.espdl_b200_arena_free(own)
        self._peer, self._turn = {}, {}
