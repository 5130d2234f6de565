"""Host side of the FP8-encoded allreduce (one process per GPU).

The reference project names this path (an FP8 allreduce over mscclpp) but holds
no code for it; the semantics are those of the configuration text: per-128
element e4m3fn blocks with an fp32 scale amax/448, fp32 accumulation in rank
order, one bf16 rounding, identical bits on every rank.  ``torch.distributed``
is used only to exchange the 64-byte IPC handles of the workspaces at set-up;
the data path is the library's own kernels storing into peer memory.
"""
from __future__ import annotations

import ctypes as C

import torch

from ._lib import check, lib

GROUP = 512          # elements per unit of ownership (4 blocks of 128)
ONE_SHOT, TWO_SHOT, AUTO = 1, 2, 0
TWO_SHOT_FP8_GATHER = 3   # all-gather re-encoded in FP8: result = decode(encode(two-shot result)); opt-in


def shard_groups(n: int, world: int):
    """[(first_group, end_group)] per rank: which 512-element groups of an
    n-element vector each rank reduces in the two-shot algorithm."""
    groups = (n + GROUP - 1) // GROUP
    return [(groups * r // world, groups * (r + 1) // world) for r in range(world)]


def quantize_blocks128(x: torch.Tensor):
    """Device encoder: (q uint8 like x, scales fp32 [numel/128]) of a bf16 tensor."""
    assert x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous() and x.numel() % 128 == 0
    q = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    s = torch.empty(x.numel() // 128, dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        check(lib().rdb_quantize_blocks128(x.data_ptr(), q.data_ptr(), s.data_ptr(), x.numel(),
                                           torch.cuda.current_stream(x.device).cuda_stream), "rdb_quantize_blocks128")
    return q, s


class _Workspace:
    def __init__(self, world: int, max_elems: int, nbytes: int | None = None):
        self.bytes = int(lib().rdb_ar_workspace_bytes(world, max_elems)) if nbytes is None else int(nbytes)
        if self.bytes == 0:
            raise ValueError("world must be 1..8 and max_elems positive")
        p = C.c_void_p()
        check(lib().rdb_ar_workspace_alloc(self.bytes, C.byref(p)), "rdb_ar_workspace_alloc")
        self.ptr = p.value

    def handle(self) -> bytes:
        buf = C.create_string_buffer(64)
        check(lib().rdb_ar_ipc_export(self.ptr, buf), "rdb_ar_ipc_export")
        return buf.raw

    def free(self):
        if self.ptr:
            lib().rdb_ar_workspace_free(self.ptr)
            self.ptr = None


def _create(rank: int, world: int, ptrs, max_elems: int) -> int:
    arr = (C.c_void_p * world)(*ptrs)
    ctx = C.c_void_p()
    check(lib().rdb_ar_create(rank, world, arr, max_elems, C.byref(ctx)), "rdb_ar_create")
    return ctx.value


class _DeviceView:
    """Lets torch wrap a raw device address (no copy, no ownership)."""

    def __init__(self, ptr: int, nelems: int):
        self.__cuda_array_interface__ = {"shape": (nelems,), "typestr": "<i2", "data": (ptr, False), "version": 3}


class Fp8AllReduce:
    """Collective object of one rank.  ``all_reduce(x)`` must be called by
    every rank of the group with tensors of the same size.

    backend="ipc": workspaces from cudaMalloc, shared through CUDA IPC handles
    (any process group can carry the 64-byte handles).  backend="symm": the
    workspace is a torch symmetric-memory allocation (needs an NCCL group);
    if the allocation has an NVLS multicast address the bf16 all-gather uses
    multimem stores.  backend="auto" tries "symm" and falls back to "ipc".

    capturable=True (every rank alike): the calls are counted on the device
    (rdb_ar_set_device_epoch), so ``all_reduce`` and ``skinny_gemm_all_reduce``
    may be recorded under ``torch.cuda.graph`` and replayed; make one call
    before the first capture and keep all calls of the object stream-ordered.
    """

    def __init__(self, max_elems: int, group=None, device=None, backend: str = "ipc", multimem: bool | None = None,
                 capturable: bool = False):
        import torch.distributed as dist
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.max_elems = int(max_elems)
        self.peers, self.ws, self.symm, self.multicast = [], None, None, False
        self.reg_ws, self.reg_symm = None, None
        nbytes = int(lib().rdb_ar_workspace_bytes(self.world, self.max_elems))
        if nbytes == 0:
            raise ValueError("world must be 1..8 and max_elems positive")
        with torch.cuda.device(self.device):
            ptrs = mc = None
            # "auto": CUDA IPC unless the multimem all-gather is asked for (it needs the multicast address of a
            # symmetric-memory allocation); with a symmetric-memory workspace the plain copy-out was measured
            # 10 us slower at 2 MiB and, once, 75 us slower at 16 MiB on 8 GPUs
            if backend == "symm" or (backend == "auto" and multimem):
                try:
                    ptrs, mc = self._symm_workspace(nbytes, dist)
                except Exception:  # noqa: BLE001
                    if backend == "symm":
                        raise
            if ptrs is None:
                ptrs = self._ipc_workspace(dist)
            self.backend = "symm" if self.symm is not None else "ipc"
            self.ctx = _create(self.rank, self.world, ptrs, self.max_elems)
            self.capturable = bool(capturable)
            if self.capturable:
                check(lib().rdb_ar_set_device_epoch(self.ctx, 1), "rdb_ar_set_device_epoch")
            if multimem is None:
                # one multicast store replaces W-1 peer stores: measured slower than per-peer stores at 2
                # and 4 ranks, 1.5 % faster at 8 ranks for 64 MiB but twice as slow there for 16 MiB with a
                # copy-out - so it is opt-in
                multimem = False
            if mc and multimem:
                check(lib().rdb_ar_set_multicast(self.ctx, mc), "rdb_ar_set_multicast")
                self.multicast = True
        dist.barrier(group=group)

    def _ipc_workspace(self, dist):
        self.ws = _Workspace(self.world, self.max_elems)
        handles = [None] * self.world
        dist.all_gather_object(handles, self.ws.handle(), group=self.group)
        ptrs = []
        for r, h in enumerate(handles):
            if r == self.rank:
                ptrs.append(self.ws.ptr)
                continue
            p = C.c_void_p()
            check(lib().rdb_ar_ipc_import(h, C.byref(p)), "rdb_ar_ipc_import")
            self.peers.append(p.value)
            ptrs.append(p.value)
        return ptrs

    def _symm_workspace(self, nbytes, dist):
        import torch.distributed._symmetric_memory as symm_mem
        grp = self.group if self.group is not None else dist.group.WORLD
        buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=self.device)
        hdl = symm_mem.rendezvous(buf, grp)
        buf.zero_()
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        self.symm = (buf, hdl)
        mc = int(getattr(hdl, "multicast_ptr", 0) or 0)
        return [int(p) for p in hdl.buffer_ptrs], mc

    def new_result_buffer(self, nelems: int) -> torch.Tensor:
        """Collective: a bf16 tensor of `nelems` elements that every rank can
        store into, registered with the context (rdb_ar_register_buffers).  A
        two-shot ``all_reduce(x, out=<this tensor or a leading slice of it>)``
        then delivers the reduced shards straight into every rank's tensor -
        no copy out of the workspace.  One registered buffer per object; a
        second call replaces the first.  Its contents are valid until work
        queued after this rank's next call."""
        import torch.distributed as dist
        nbytes = (int(nelems) * 2 + 255) // 256 * 256
        with torch.cuda.device(self.device):
            self._drop_result_buffer()
            if self.backend == "symm":
                import torch.distributed._symmetric_memory as symm_mem
                grp = self.group if self.group is not None else dist.group.WORLD
                buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=self.device)
                hdl = symm_mem.rendezvous(buf, grp)
                self.reg_symm = (buf, hdl)
                ptrs, own = [int(p) for p in hdl.buffer_ptrs], buf.data_ptr()
            else:
                self.reg_ws = _Workspace(self.world, 0, nbytes=nbytes)
                handles = [None] * self.world
                dist.all_gather_object(handles, self.reg_ws.handle(), group=self.group)
                ptrs, self.reg_peers = [], []
                for r, h in enumerate(handles):
                    if r == self.rank:
                        ptrs.append(self.reg_ws.ptr)
                        continue
                    p = C.c_void_p()
                    check(lib().rdb_ar_ipc_import(h, C.byref(p)), "rdb_ar_ipc_import")
                    self.reg_peers.append(p.value)
                    ptrs.append(p.value)
                own = self.reg_ws.ptr
            arr = (C.c_void_p * self.world)(*ptrs)
            check(lib().rdb_ar_register_buffers(self.ctx, arr, nbytes), "rdb_ar_register_buffers")
            dist.barrier(group=self.group)
            return torch.as_tensor(_DeviceView(own, int(nelems)), device=self.device).view(torch.bfloat16)

    def _drop_result_buffer(self):
        if self.reg_ws is None and self.reg_symm is None:
            return
        torch.cuda.synchronize(self.device)
        if getattr(self, "ctx", None):
            lib().rdb_ar_register_buffers(self.ctx, None, 0)
        for p in getattr(self, "reg_peers", []):
            lib().rdb_ar_ipc_close(p)
        self.reg_peers = []
        if self.reg_ws is not None:
            self.reg_ws.free()
        self.reg_ws, self.reg_symm = None, None

    def all_reduce(self, x: torch.Tensor, out: torch.Tensor | None = None, algo: int = AUTO,
                   check_status: bool = False) -> torch.Tensor:
        """``check_status=True`` synchronises the device after the call and
        raises if a bounded wait ran out (this rank's, or one a peer reported):
        ``out`` is not valid then.  Without it the call is asynchronous and the
        caller reads ``rdb_device_status()`` when it next synchronises."""
        assert x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous()
        n = x.numel()
        if out is None:
            out = torch.empty_like(x)
        assert out.dtype == torch.bfloat16 and out.is_contiguous() and out.numel() == n
        # a small call is a few microseconds of device time: keep the host path short (no device-context switch when
        # this rank's device is already current)
        if torch.cuda.current_device() == self.device.index:
            code = lib().rdb_ar_allreduce(self.ctx, x.data_ptr(), out.data_ptr(), n, algo,
                                          torch.cuda.current_stream().cuda_stream)
        else:
            with torch.cuda.device(self.device):
                code = lib().rdb_ar_allreduce(self.ctx, x.data_ptr(), out.data_ptr(), n, algo,
                                              torch.cuda.current_stream(self.device).cuda_stream)
        if code != 0:
            check(code, "rdb_ar_allreduce")
        if check_status:
            with torch.cuda.device(self.device):
                check(lib().rdb_device_status(), "rdb_ar_allreduce (device status)")
        return out

    def skinny_gemm_all_reduce(self, A: torch.Tensor, B: torch.Tensor, scale_a: torch.Tensor, scale_b: torch.Tensor,
                               out: torch.Tensor | None = None) -> torch.Tensor:
        """Row-parallel linear + allreduce (rdb_skinny_gemm_fp8_allreduce): this
        rank's K slice ``A [M,K_r]``, ``B [N,K_r]`` is multiplied and the bf16
        partial product goes, block-quantised by the GEMM's epilogue, straight
        into every rank's staging area; the result ``[M,N]`` bf16 is the
        FP8-encoded allreduce of the ranks' partial products.  N % 128 == 0,
        M * N <= 2**20."""
        from .skinny_gemm import _problem_array
        M, N = A.shape[0], B.shape[0]
        if out is None:
            out = torch.empty((M, N), dtype=torch.bfloat16, device=self.device)
        assert out.dtype == torch.bfloat16 and out.is_contiguous() and out.numel() == M * N
        arr = _problem_array([(A, B, scale_a, scale_b, out)])      # D of the problem is not written by the fused call
        with torch.cuda.device(self.device):
            check(lib().rdb_skinny_gemm_fp8_allreduce(self.ctx, arr, out.data_ptr(),
                                                      torch.cuda.current_stream(self.device).cuda_stream),
                  "rdb_skinny_gemm_fp8_allreduce")
        return out

    def all_reduce_in_workspace(self, x: torch.Tensor) -> torch.Tensor:
        """Two-shot allreduce whose result is left in the workspace: returns a
        bf16 view of it (no copy-out), valid until this rank's next call."""
        assert x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous()
        n = x.numel()
        with torch.cuda.device(self.device):
            check(lib().rdb_ar_allreduce(self.ctx, x.data_ptr(), None, n, TWO_SHOT,
                                         torch.cuda.current_stream(self.device).cuda_stream), "rdb_ar_allreduce")
            ptr = int(lib().rdb_ar_result(self.ctx))
            return torch.as_tensor(_DeviceView(ptr, n), device=self.device).view(torch.bfloat16)

    def close(self):
        if getattr(self, "ctx", None):
            torch.cuda.synchronize(self.device)
            self._drop_result_buffer()
            lib().rdb_ar_destroy(self.ctx)
            self.ctx = None
            for p in self.peers:
                lib().rdb_ar_ipc_close(p)
            if self.ws is not None:
                self.ws.free()
            self.symm = None


class LocalRanks:
    """W ranks emulated on ONE GPU (tests and single-GPU drivers): W
    workspaces on the same device, and each phase issued for every rank before
    the next phase of any, so that no launch waits on one not yet issued."""

    def __init__(self, world: int, max_elems: int, device="cuda"):
        self.world, self.device = world, torch.device(device)
        with torch.cuda.device(self.device):
            self.ws = [_Workspace(world, max_elems) for _ in range(world)]
            ptrs = [w.ptr for w in self.ws]
            self.ctx = [_create(r, world, ptrs, max_elems) for r in range(world)]
        self.reg = []

    def new_result_buffers(self, nelems: int):
        """One registered result buffer per emulated rank (see
        Fp8AllReduce.new_result_buffer); returns the W bf16 tensors."""
        nbytes = (int(nelems) * 2 + 255) // 256 * 256
        with torch.cuda.device(self.device):
            self.reg = [_Workspace(self.world, 0, nbytes=nbytes) for _ in range(self.world)]
            arr = (C.c_void_p * self.world)(*[w.ptr for w in self.reg])
            for c in self.ctx:
                check(lib().rdb_ar_register_buffers(c, arr, nbytes), "rdb_ar_register_buffers")
            return [torch.as_tensor(_DeviceView(w.ptr, int(nelems)), device=self.device).view(torch.bfloat16)
                    for w in self.reg]

    def all_reduce(self, xs, algo: int = AUTO, outs=None):
        """xs: list of W bf16 tensors (one per emulated rank) -> list of W results."""
        n = xs[0].numel()
        if outs is None:
            outs = [torch.empty_like(x) for x in xs]
        stream = torch.cuda.current_stream(self.device).cuda_stream
        with torch.cuda.device(self.device):
            epochs = {int(lib().rdb_ar_begin_call(c)) for c in self.ctx}
            assert len(epochs) == 1
            epoch = epochs.pop()
            for phase in (1, 2, 3):
                for r in range(self.world):
                    check(lib().rdb_ar_phase(self.ctx[r], phase, epoch, xs[r].data_ptr(), outs[r].data_ptr(), n, algo,
                                             stream), "rdb_ar_phase")
        return outs

    def skinny_gemm_all_reduce(self, operands):
        """operands: per emulated rank (A_r, B_r, scale_a, scale_b).  The
        producer launches of all ranks first, then the consuming ones."""
        from .skinny_gemm import _problem_array
        M, N = operands[0][0].shape[0], operands[0][1].shape[0]
        outs = [torch.empty((M, N), dtype=torch.bfloat16, device=self.device) for _ in operands]
        stream = torch.cuda.current_stream(self.device).cuda_stream
        with torch.cuda.device(self.device):
            for r, (A, B, sa, sb) in enumerate(operands):
                check(lib().rdb_skinny_gemm_fp8_allreduce_begin(self.ctx[r], _problem_array([(A, B, sa, sb, outs[r])]), stream),
                      "rdb_skinny_gemm_fp8_allreduce_begin")
            for r in range(self.world):
                check(lib().rdb_skinny_gemm_fp8_allreduce_finish(self.ctx[r], outs[r].data_ptr(), stream),
                      "rdb_skinny_gemm_fp8_allreduce_finish")
        return outs

    def close(self):
        torch.cuda.synchronize(self.device)
        for c in self.ctx:
            lib().rdb_ar_destroy(c)
        for w in self.ws + self.reg:
            w.free()
        self.ctx, self.ws, self.reg = [], [], []
