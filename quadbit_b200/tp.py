"""Peer-mapped buffers and flag words for tensor parallelism on one NVSwitch box (one process per GPU).

`PeerBuffer` is one device allocation per rank whose address is exchanged as a CUDA IPC handle, so every rank holds a
pointer to every other rank's copy; the fused kernels (`qb_gemm_rs`, `qb_reduce_norm_quant`) store straight into those
pointers. `TPContext` owns the buffers one model needs: two sets of reduce-scatter slots, two gathered activation
arrays and the flag words that order producers and consumers across GPUs.

With `emulate=n` all n "ranks" live in this process on one GPU (plain device pointers instead of IPC): the data path of
the multi-GPU kernels then runs on a single GPU, rank by rank in stream order (a producer kernel is always launched before
the consumer that waits for it, so nothing spins on work that has not been submitted)."""
from __future__ import annotations

import ctypes

import torch

from ._lib import check, load


class _RawCuda:
    """Minimal __cuda_array_interface__ holder so torch can view a raw device pointer."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3, "strides": None}


def view_u8(ptr: int, nbytes: int, device) -> torch.Tensor:
    return torch.as_tensor(_RawCuda(ptr, nbytes), device=device)


class PeerBuffer:
    """`nbytes` zero-filled bytes on every rank; `ptrs[r]` is rank r's buffer as seen from this process."""

    def __init__(self, nbytes: int, rank: int, world: int, group=None, device=None):
        import torch.distributed as dist
        self.lib = lib = load("sparse_fp4")
        self.nbytes, self.rank, self.world = int(nbytes), rank, world
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        p = ctypes.c_void_p()
        check(lib.qb_peer_alloc(ctypes.byref(p), self.nbytes), "qb_peer_alloc")
        self.own = p.value
        self.ptrs = [0] * world
        self.ptrs[rank] = self.own
        self._opened = []
        if world > 1:
            h = ctypes.create_string_buffer(64)
            rc = lib.qb_peer_export(self.own, h)
            handles = [None] * world
            dist.all_gather_object(handles, (rc, bytes(h.raw)), group=group)
            err = max(hr[0] for hr in handles)
            if not err:
                for r in range(world):
                    if r == rank:
                        continue
                    q = ctypes.c_void_p()
                    err = lib.qb_peer_open(ctypes.create_string_buffer(handles[r][1], 64), ctypes.byref(q))
                    if err:
                        break
                    self.ptrs[r] = q.value
                    self._opened.append(q.value)
            # all ranks agree on the outcome, so a refusal on one rank raises on every rank at the same point
            errs = [None] * world
            dist.all_gather_object(errs, int(err), group=group)
            if any(errs):
                self.close()
                raise RuntimeError(f"peer mapping failed (CUDA IPC codes per rank: {errs})")
        self.tensor = view_u8(self.own, self.nbytes, self.device)       # this rank's copy as a torch tensor (uint8)

    def close(self):
        for q in self._opened:
            self.lib.qb_peer_close(q)
        self._opened = []
        if self.own:
            self.lib.qb_peer_free(self.own)
            self.own = 0


class _EmulatedPeers:
    """n buffers in one process: ptrs are plain device pointers."""

    def __init__(self, nbytes: int, n: int, device):
        self.tensors = [torch.zeros(int(nbytes), dtype=torch.uint8, device=device) for _ in range(n)]
        self.ptrs = [t.data_ptr() for t in self.tensors]


def ptr_array(ptrs):
    return (ctypes.c_void_p * len(ptrs))(*ptrs)


def _align(x, a=256):
    return (x + a - 1) // a * a


class TPContext:
    """Buffers of one tensor-parallel model instance for `T` tokens of hidden size `H`.

    slots[k]      reduce-scatter destinations (k = 0 after o_proj, 1 after down): [world][T/world][H] bf16 on every rank;
                  rank s stores its partial rows of rank r's token range into r's slot s.
    gathered[b]   quantised activations of all T tokens on every rank (b = 16 dense / 32 sparse input): packed bytes
                  [T][H/2], scale atoms, globals [T]; every rank stores its rows into all copies.
    flags         four arrays of `world` ints on every rank (slots 0 / 1 landed, gathered 16 / 32 landed), written with
                  the value of `epoch`, a device counter that every rank bumps once per layer (equal on all ranks).
    """

    FLAG_SLOT = (0, 1)
    FLAG_GATHER = {16: 2, 32: 3}

    def __init__(self, T: int, H: int, rank: int, world: int, group=None, device=None, emulate=None):
        self.lib = lib = load("sparse_fp4")
        self.T, self.H, self.rank, self.world = T, H, rank, world
        assert T % (128 * world) == 0, "tokens per rank must be a multiple of 128 (scale-factor atoms are 128 rows)"
        self.Tl = T // world
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.slot_bytes = _align(world * self.Tl * H * 2)
        self.g_off = {}
        self.g_bytes = {}
        for b in (16, 32):
            o_sf = _align(T * H // 2)
            o_g = o_sf + _align(lib.qb_sf_atoms_bytes(T, H, b))
            self.g_off[b] = (0, o_sf, o_g)
            self.g_bytes[b] = o_g + _align(T * 4)
        sizes = [self.slot_bytes, self.slot_bytes, self.g_bytes[16], self.g_bytes[32], 4096]
        if emulate is not None:
            self.bufs = emulate          # shared list of _EmulatedPeers, one per buffer kind
        else:
            self.bufs = [PeerBuffer(n, rank, world, group, self.device) for n in sizes]
        self.sizes = sizes
        self.done = torch.zeros(16, dtype=torch.int32, device=self.device)
        # Flag values are the "epoch", a device word every rank bumps at the same points of its stream (qb_epoch_add): the
        # kernels read it when they run, so their arguments never change and a whole forward can be replayed from a CUDA
        # graph. It starts at 1: the flag words start at 0 and the first wait must not pass on that.
        self.epoch = torch.ones(1, dtype=torch.int32, device=self.device)

    @staticmethod
    def emulated(T: int, H: int, world: int, device):
        """`world` contexts sharing one GPU (buffers are plain allocations of this process)."""
        lib = load("sparse_fp4")
        slot = _align(T * H * 2)
        g = {b: _align(T * H // 2) + _align(lib.qb_sf_atoms_bytes(T, H, b)) + _align(T * 4) for b in (16, 32)}
        shared = [_EmulatedPeers(n, world, device) for n in (slot, slot, g[16], g[32], 4096)]
        return [TPContext(T, H, r, world, device=device, emulate=shared) for r in range(world)]

    # ---- addresses
    def own_tensor(self, k: int) -> torch.Tensor:
        b = self.bufs[k]
        return b.tensors[self.rank] if isinstance(b, _EmulatedPeers) else b.tensor

    def slot_out_ptrs(self, k: int):
        """Where this rank's GEMM epilogue stores the rows of every owner: owner r's slot `rank`."""
        off = self.rank * self.Tl * self.H * 2
        return ptr_array([p + off for p in self.bufs[k].ptrs])

    def slots_view(self, k: int) -> torch.Tensor:
        """This rank's slots [world][Tl][H] bf16."""
        return self.own_tensor(k)[: self.world * self.Tl * self.H * 2].view(torch.bfloat16).view(self.world, self.Tl, self.H)

    def gathered_ptrs(self, block: int):
        k = 2 if block == 16 else 3
        o_b, o_sf, o_g = self.g_off[block]
        ps = self.bufs[k].ptrs
        return ptr_array([p + o_b for p in ps]), ptr_array([p + o_sf for p in ps]), ptr_array([p + o_g for p in ps])

    def gathered_own(self, block: int):
        """(Bbytes ptr, atoms ptr, g ptr) of this rank's gathered arrays."""
        k = 2 if block == 16 else 3
        o_b, o_sf, o_g = self.g_off[block]
        p = self.bufs[k].ptrs[self.rank]
        return p + o_b, p + o_sf, p + o_g

    def flag_ptrs(self, which: int):
        """Flag array `which` of every rank."""
        return ptr_array([p + which * 64 for p in self.bufs[4].ptrs])

    def flag_own(self, which: int) -> int:
        return self.bufs[4].ptrs[self.rank] + which * 64

    def bump(self, stream: int):
        check(self.lib.qb_epoch_add(self.epoch.data_ptr(), 1, stream), "qb_epoch_add")

    def close(self):
        for b in self.bufs:
            if isinstance(b, PeerBuffer):
                b.close()


class EPContext:
    """Peer buffers of one expert-parallel MoE layer instance: `T` tokens in total (T / world per rank, rows of `x_width`
    bf16 values as the gather reads them), `topk` slots per token, `r_cap` routed rows of capacity and `mpe_dn` output
    features per routed row on every rank.

    x_pub     this rank's token rows, readable by every rank (the owner of an expert pulls the rows it needs);
    tables    the routing of ALL tokens, replicated on every rank by peer stores: expert ids [T*topk] i64, weights f32;
    d         weighted expert outputs of this rank's experts [r_cap][mpe_dn] bf16, read by the tokens' home ranks;
    inverse   row of every slot in `d` (-1 for slots of other ranks' experts) [T*topk] i32, read by the home ranks;
    flags     two arrays of `world` ints (tables published, outputs ready), values = the device epoch."""

    FLAG_PUBLISHED, FLAG_OUTPUT = 0, 1

    def __init__(self, T: int, x_width: int, topk: int, mpe_dn: int, r_cap: int, rank: int, world: int, group=None, device=None,
                 emulate=None):
        self.lib = load("sparse_fp4")
        assert T % world == 0
        self.T, self.Tl, self.topk, self.rank, self.world = T, T // world, topk, rank, world
        self.x_width, self.mpe_dn, self.r_cap = x_width, mpe_dn, r_cap
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        n = T * topk
        self.off_w = _align(n * 8)
        self.sizes = [_align(self.Tl * x_width * 2), self.off_w + _align(n * 4), _align(r_cap * mpe_dn * 2), _align(n * 4), 4096]
        self.bufs = emulate if emulate is not None else [PeerBuffer(b, rank, world, group, self.device) for b in self.sizes]
        self.done = torch.zeros(4, dtype=torch.int32, device=self.device)
        self.epoch = torch.ones(1, dtype=torch.int32, device=self.device)

    @staticmethod
    def emulated(T, x_width, topk, mpe_dn, r_cap, world, device):
        probe = [_align(T // world * x_width * 2), _align(T * topk * 8) + _align(T * topk * 4), _align(r_cap * mpe_dn * 2),
                 _align(T * topk * 4), 4096]
        shared = [_EmulatedPeers(b, world, device) for b in probe]
        return [EPContext(T, x_width, topk, mpe_dn, r_cap, r, world, device=device, emulate=shared) for r in range(world)]

    def ptrs(self, k: int, off: int = 0):
        return ptr_array([p + off for p in self.bufs[k].ptrs])

    def own(self, k: int, off: int = 0) -> int:
        return self.bufs[k].ptrs[self.rank] + off

    def own_tensor(self, k: int) -> torch.Tensor:
        b = self.bufs[k]
        return b.tensors[self.rank] if isinstance(b, _EmulatedPeers) else b.tensor

    def flag_ptrs(self, which: int):
        return self.ptrs(4, which * 64)

    def flag_own(self, which: int) -> int:
        return self.own(4, which * 64)

    def bump(self, stream: int):
        check(self.lib.qb_epoch_add(self.epoch.data_ptr(), 1, stream), "qb_epoch_add")

    def close(self):
        for b in self.bufs:
            if isinstance(b, PeerBuffer):
                b.close()
