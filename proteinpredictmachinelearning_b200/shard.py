"""Partition of the contraction ops over the GPUs of one box (one process per GPU).

Every activation is split into `world` contiguous chunks of its flat buffer, which under the
reference's flat-buffer semantics means: token rows for mul_mat / Q8 mul_mat and attention batches,
channel slabs d for the triangle multiplication (flat [D][I][K]: D independent L x L matrices,
src/backend/CPUKernels.cpp:934-957) and left-channel slabs d1 for the outer-product-mean (flat
[D][L][N]: output block (d1, d2) needs slab d1 of `left` and all of `right`,
src/backend/CPUKernels.cpp:1022-1028).  Only the outer-product-mean needs an exchange (all-gather of
`right`); everything else is rank-local."""


def split(total, world, rank, align=1):
    """Contiguous [lo, hi) of `total` units for `rank`; boundaries are multiples of `align`
    (the last shard takes the remainder)."""
    if world <= 0 or not (0 <= rank < world) or total < 0 or align <= 0:
        raise ValueError("bad shard arguments")
    units = (total + align - 1) // align
    per = (units + world - 1) // world
    lo = min(rank * per * align, total)
    hi = min((rank + 1) * per * align, total)
    return lo, hi


def token_rows(M, world, rank):
    """mul_mat / Q8 mul_mat: rows of X (tokens) are independent."""
    return split(M, world, rank)


def attention_batches(B, world, rank):
    """OP_FLASH_ATTN_EXT: the outer batch B' (MSA rows, pair rows) is independent."""
    return split(B, world, rank)


def tri_mul_slabs(D, world, rank):
    """OP_TRI_MUL: channel slabs."""
    return split(D, world, rank)


def opm_slabs(D, world, rank):
    """OP_OUTER_PROD_MEAN: the d1 range of the output this rank owns (needs all of `right`)."""
    return split(D, world, rank)


def _require_equal_shards(n_local, world, group, what):
    """Every rank must bring the same number of leading rows: a collective entered with different sizes hangs or
    overwrites memory.  The sizes are exchanged first (one small all-gather) and a mismatch raises on every rank."""
    import torch
    import torch.distributed as dist
    mine = torch.tensor([int(n_local)], dtype=torch.int64)
    backend = dist.get_backend(group)
    if backend == "nccl":
        mine = mine.cuda()
    sizes = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(sizes, mine, group=group)
    sizes = [int(t.item()) for t in sizes]
    if any(n != sizes[0] for n in sizes):
        raise ValueError(f"{what}: ranks hold different shard sizes {sizes}; split a total that is a multiple of the "
                         "number of ranks (split(total, world, rank) gives the last rank the remainder otherwise)")


def all_gather_rows(x_local, world, group=None):
    """All-gather along dim 0 of equally sized shards (NCCL on GPUs, gloo in the CPU tests).  Raises ValueError on
    every rank when the shards differ in size."""
    import torch
    import torch.distributed as dist
    if world == 1:
        return x_local
    _require_equal_shards(x_local.shape[0], world, group, "all_gather_rows")
    parts = [torch.empty_like(x_local) for _ in range(world)]
    dist.all_gather(parts, x_local.contiguous(), group=group)
    return torch.cat(parts, dim=0)


def transpose_exchange(x_local, world, group=None):
    """The (n, l) transpose of an activation [N, L, C] that is sharded by contiguous n ranges, as the reference's
    `permute({0,2,1,3})` copies after MSA column attention and pair row attention do on one device
    (src/modules/Attention.cpp:489, :744): x_local [N/world, L, C] -> this rank's rows [L/world, N, C] of the transposed
    tensor.  One all-to-all in which every rank keeps 1/world of its data, plus local re-layouts."""
    import torch.distributed as dist
    n_loc, L, C = x_local.shape
    if world == 1:
        return x_local.permute(1, 0, 2).contiguous()
    if L % world:
        raise ValueError("L must be a multiple of the number of ranks")
    _require_equal_shards(n_loc, world, group, "transpose_exchange")
    l_loc = L // world
    send = x_local.reshape(n_loc, world, l_loc, C).permute(1, 0, 2, 3).contiguous()      # [to rank][n][l][c]
    recv = send.new_empty(send.shape)                                                    # [from rank][n][l][c]
    dist.all_to_all_single(recv, send, group=group)
    return recv.permute(2, 0, 1, 3).reshape(l_loc, world * n_loc, C).contiguous()


class PeerBuffers:
    """Device buffers that the other ranks of the box write into directly (csrc/peer_exchange.cu): allocated by the
    library, shared once through CUDA IPC handles sent over the process group, wrapped as torch tensors for local use."""

    def __init__(self, world, rank, group=None):
        import ctypes as C
        from . import _lib
        self.C, self.lib = C, _lib.load()
        self.world, self.rank, self.group = world, rank, group
        self.local, self.mapped = [], []
        self.flags = self._share(self.lib.ppml_b200_peer_flag_bytes())

    def _share(self, nbytes):
        """Allocates `nbytes` here, maps every peer's allocation of the same call; returns (local pointer, ctypes array of
        `world` pointers with entry `rank` = local)."""
        import torch.distributed as dist
        C = self.C
        p = self.lib.ppml_b200_peer_alloc(int(nbytes))
        if not p:
            raise RuntimeError("peer_alloc failed")
        self.local.append(p)
        ptrs = [None] * self.world
        ptrs[self.rank] = p
        if self.world > 1:
            h = C.create_string_buffer(64)
            if self.lib.ppml_b200_peer_export(C.c_void_p(p), h) != 0:
                raise RuntimeError("peer_export failed")
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(h.raw), group=self.group)
            for r in range(self.world):
                if r != self.rank:
                    q = self.lib.ppml_b200_peer_open(C.create_string_buffer(handles[r], 64))
                    if not q:
                        raise RuntimeError(f"peer_open failed for rank {r}")
                    self.mapped.append(q)
                    ptrs[r] = q
        return p, (C.c_void_p * self.world)(*ptrs)

    def tensor(self, shape, dtype=None):
        """A zero-filled fp32 tensor in shared memory: (local torch view, peer pointer array)."""
        import math
        import torch
        nbytes = 4 * math.prod(shape)
        p, arr = self._share((nbytes + 255) // 256 * 256)

        class _Raw:
            __cuda_array_interface__ = {"shape": tuple(shape), "typestr": "<f4", "data": (p, False), "version": 2}
        return torch.as_tensor(_Raw(), device="cuda"), arr

    def _stream(self, stream):
        import torch
        if stream is not None:
            return stream
        s = torch.cuda.current_stream().cuda_stream       # the capture stream while a CUDA graph is being recorded
        return self.C.c_void_p(s) if s else None

    def all_gather(self, x, dst_ptrs, site, stream=None):
        stream = self._stream(stream)
        rc = self.lib.ppml_b200_peer_all_gather(self.C.c_void_p(x.data_ptr()), dst_ptrs, x.numel() * x.element_size(), self.rank, self.world,
                                                self.flags[1], site, stream)
        if rc != 0:
            raise RuntimeError(f"peer_all_gather failed with status {rc}")

    def transpose(self, x, out_ptrs, n_loc, L, Cc, site, stream=None):
        stream = self._stream(stream)
        rc = self.lib.ppml_b200_peer_transpose(self.C.c_void_p(x.data_ptr()), out_ptrs, n_loc, L, Cc, self.rank, self.world,
                                               self.flags[1], site, stream)
        if rc != 0:
            raise RuntimeError(f"peer_transpose failed with status {rc}")

    def close(self):
        for q in self.mapped:
            self.lib.ppml_b200_peer_close(self.C.c_void_p(q))
        for p in self.local:
            self.lib.ppml_b200_peer_free(self.C.c_void_p(p))
        self.mapped, self.local = [], []
