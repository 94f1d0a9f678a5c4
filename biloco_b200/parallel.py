"""Tensor-parallel use of the fused linear on the GPUs of one box (one process per GPU, torch.distributed).

The path shards without an exchange inside the kernel:

  * column-parallel (N split): rank g keeps rows [g*N/G, (g+1)*N/G) of the residual (codes + block scales) and of U, the
    whole of V and the coefficients. Outputs stay sharded; the z stage is recomputed identically on every rank.
  * row-parallel (K split): rank g keeps columns [g*K/G, (g+1)*K/G) of the residual and rows of V, the whole of U. Each
    rank's launch yields a partial y over all N (its K-slice of the FP4 product plus U . (S * V_g^T x_g), both linear
    in the K-slice), and ONE all-reduce (NCCL over NVLink) of the [M, N] outputs finishes the layer.

The NVFP4 tensor scale of an activation is defined over the whole [tokens, K] tensor; ranks that hold K-slices agree on
it with a one-float max all-reduce before quantising (`agree_on_activation_scale`), so the codes equal the single-GPU
ones. With ``local_scale=True`` every rank scales its own K-slice instead (its partial sum carries its own decode
scale, so the sum is still the layer's output; the codes then differ from the single-GPU ones, within the same
tolerance): one collective and half a dozen small kernels less per call, which is what a decode step wants. The reference has no distributed code; this is the N/K sharding that BASELINE configs 3 and 4 ask for.
"""
import torch
import torch.distributed as dist


def shard_bounds(n: int, world: int, rank: int, multiple: int):
    """[lo, hi) of rank's equal share of n; n / world must be a multiple of `multiple`."""
    assert n % world == 0 and (n // world) % multiple == 0, f"{n} does not split into {world} shards of a multiple of {multiple}"
    per = n // world
    return rank * per, (rank + 1) * per


def _sf_view(W_sf, N, K):
    """Block scales in the 128x4 atom layout as [N/128, K/64, 32, 4, 4] = (row block, k atom, row%32, row/32%4, kblock%4)."""
    return W_sf.view(torch.uint8).reshape(-1)[: ((N + 127) // 128 * 128) * (K // 16)].view((N + 127) // 128, K // 64, 32, 4, 4)


def shard_column_parallel(ops: dict, world: int, rank: int):
    """Operands of rank's N-shard. ops: W_codes [N,K/2], W_sf (atom layout), w_gscale, V_packed [r,K/8], U_packed [r,N/8],
    S [r], smooth_scale [K], bias [N] or None."""
    N, K = ops["W_codes"].shape[0], ops["W_codes"].shape[1] * 2
    lo, hi = shard_bounds(N, world, rank, 128)
    sf = _sf_view(ops["W_sf"], N, K)[lo // 128: hi // 128].contiguous().reshape(-1)
    out = dict(ops)
    out.update(W_codes=ops["W_codes"][lo:hi].contiguous(), W_sf=sf.view(ops["W_sf"].dtype),
               U_packed=ops["U_packed"][:, lo // 8: hi // 8].contiguous(),
               bias=None if ops.get("bias") is None else ops["bias"][lo:hi].contiguous())
    return out


def shard_row_parallel(ops: dict, world: int, rank: int):
    """Operands of rank's K-shard (the bias stays with rank 0 so that the all-reduce adds it once)."""
    N, K = ops["W_codes"].shape[0], ops["W_codes"].shape[1] * 2
    lo, hi = shard_bounds(K, world, rank, 256)
    sf = _sf_view(ops["W_sf"], N, K)[:, lo // 64: hi // 64].contiguous().reshape(-1)
    out = dict(ops)
    out.update(W_codes=ops["W_codes"][:, lo // 2: hi // 2].contiguous(), W_sf=sf.view(ops["W_sf"].dtype),
               V_packed=ops["V_packed"][:, lo // 8: hi // 8].contiguous(),
               smooth_scale=ops["smooth_scale"][lo:hi].contiguous(),
               bias=ops.get("bias") if rank == 0 else None)
    return out


def agree_on_activation_scale(x_local: torch.Tensor, smooth_local: torch.Tensor = None, rule: str = None, group=None):
    """fp32 [1] tensor scale of the full activation whose K-slice this rank holds (max all-reduce of one float)."""
    from . import fp4
    xs = x_local.to(torch.bfloat16)
    if smooth_local is not None:
        xs = xs / smooth_local
    amax = xs.float().abs().max().reshape(1)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(amax, op=dist.ReduceOp.MAX, group=group)
    return fp4.activation_scale_from_amax(amax, rule)


class PeerAllReduce:
    """All-reduce of fp32 partial outputs over peer memory in ONE launch per rank (biloco_b200_peer_allreduce: NVLink
    stores into the peers' receive buffers, value and call number in one 8-byte word, sums in rank order, so every rank
    gets the same bits). One object per process group, shared by all its row-parallel layers: the group's calls must be
    issued in the same order on every rank, which a tensor-parallel model does. Replaces ncclAllReduce + the cast to bf16
    where the message is a decode step's [M, N] (latency-bound). No counterpart in the reference."""

    _by_group = {}

    @classmethod
    def for_group(cls, group, device, count):
        """The group's object, (re)created collectively when `count` elements do not fit its slots."""
        key = id(group) if group is not None else 0
        obj = cls._by_group.get(key)
        if obj is None or obj.slot_elems < count:
            if obj is not None:
                obj.close()
            obj = cls(group, device, max(count, 32 * 8192))
            cls._by_group[key] = obj
        return obj

    def __init__(self, group, device, slot_elems):
        import ctypes
        from . import _lib
        lib = _lib.load()
        self.group, self.device, self.slot_elems = group, torch.device(device), int(slot_elems)
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        with torch.cuda.device(self.device):
            nbytes = lib.biloco_b200_peer_buffer_bytes(self.world, self.slot_elems)
            assert nbytes > 0, "peer all-reduce: group too large"
            ptr, handle = ctypes.c_void_p(), (ctypes.c_ubyte * 64)()
            _lib.check(lib.biloco_b200_peer_buffer_create(nbytes, ctypes.byref(ptr), handle), "peer_buffer_create")
            self.local = ptr.value
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(handle), group=group)
            self.ptrs, self._opened = [], []
            for p in range(self.world):
                if p == self.rank:
                    self.ptrs.append(self.local)
                    continue
                q = ctypes.c_void_p()
                h = (ctypes.c_ubyte * 64).from_buffer_copy(handles[p])
                _lib.check(lib.biloco_b200_peer_buffer_open(h, ctypes.byref(q)), f"peer_buffer_open (rank {p})")
                self.ptrs.append(q.value)
                self._opened.append(q.value)
            self.table = torch.tensor(self.ptrs, dtype=torch.int64, device=self.device)
            self.status = torch.zeros(16, dtype=torch.int32, device=self.device)
            torch.cuda.synchronize(self.device)
        dist.barrier(group=group)          # every rank has mapped every buffer before anybody stores into one

    def push_args(self):
        """What BiLoCoGemm.peer_push takes: the fused launch's epilogue then stores its outputs into the peers' buffers itself
        (biloco_b200_fused_linear_push) and the call below only gathers (pushed=True)."""
        return (self.table.data_ptr(), self.status.data_ptr(), self.world, self.rank, self.slot_elems)

    def __call__(self, partial, residual=None, out=None, fp32_out=False, pushed=False):
        """partial fp32 (contiguous, <= slot_elems elements) -> the sum over the ranks (+ residual bf16), bf16 or fp32, same shape.
        pushed: the launch that produced `partial` has already stored it into the peers' buffers (push_args)."""
        from . import _lib
        assert partial.is_cuda and partial.dtype == torch.float32 and partial.is_contiguous() and partial.numel() <= self.slot_elems
        assert residual is None or (residual.dtype == torch.bfloat16 and residual.is_contiguous() and residual.numel() == partial.numel())
        if out is None:
            out = torch.empty(partial.shape, device=partial.device, dtype=torch.float32 if fp32_out else torch.bfloat16)
        with torch.cuda.device(self.device):
            rc = _lib.load().biloco_b200_peer_allreduce(
                partial.data_ptr(), residual.data_ptr() if residual is not None else None, out.data_ptr(), self.table.data_ptr(),
                self.status.data_ptr(), self.world, self.rank, partial.numel(), self.slot_elems, (0x400 if fp32_out else 0) | (1 if pushed else 0),
                torch.cuda.current_stream().cuda_stream)
        _lib.check(rc, "peer_allreduce")
        return out

    def failed(self) -> bool:
        """True when a poll of an earlier call ran out of its time budget (synchronises)."""
        return bool(self.status[0].item())

    def close(self):
        """Collective: unmap the peers' buffers, then free the local one."""
        from . import _lib
        lib = _lib.load()
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        with torch.cuda.device(self.device):
            for q in self._opened:
                lib.biloco_b200_peer_buffer_close(q)
            self._opened = []
            dist.barrier(group=self.group)
            if self.local:
                lib.biloco_b200_peer_buffer_destroy(self.local)
                self.local = None

    @classmethod
    def close_all(cls):
        for obj in list(cls._by_group.values()):
            obj.close()
        cls._by_group.clear()


class ShardedBiLoCoLinear:
    """One rank's shard of a quantised layer, run through the fused kernel.

    kind = "column": forward(x [M, K]) -> y [M, N/G] (local columns).
    kind = "row":    forward(x_local [M, K/G]) -> y [M, N], all-reduced over the group.
    """

    peer_allreduce = True      # row shards on CUDA under NCCL: the library's own one-launch all-reduce instead of ncclAllReduce + cast
    epilogue_push = True       # ... with the transfer started by the fused launch's own epilogue (biloco_b200_fused_linear_push)

    def __init__(self, ops: dict, kind: str, M: int, group=None, presharded: bool = False, local_scale: bool = False):
        """ops: the operands of the whole layer (sharded here), or with presharded=True this rank's shard as it is.
        local_scale (row shards): every rank quantises its K-slice with its own tensor scale (see the module text)."""
        from .kernel import BiLoCoGemm
        assert kind in ("column", "row")
        self.kind, self.M, self.group, self.local_scale = kind, M, group, local_scale
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.ops = dict(ops) if presharded else (shard_column_parallel if kind == "column" else shard_row_parallel)(ops, world, rank)
        o = self.ops
        self.N, self.K = o["W_codes"].shape[0], o["W_codes"].shape[1] * 2
        dev = o["W_codes"].device
        self.alpha = torch.zeros(1, device=dev, dtype=torch.float32)
        self.gemm = BiLoCoGemm(o["W_codes"], o["W_sf"].view(torch.float8_e4m3fn), self.alpha, o["V_packed"], o["U_packed"], o["S"], M=M,
                               back_to_back=False)
        self.gemm.fp32_out = kind == "row"     # partial sums are reduced in fp32; one bf16 rounding after the all-reduce
        if o.get("bias") is not None:
            self.gemm.residual = o["bias"].to(torch.bfloat16).unsqueeze(0).expand(M, self.N).contiguous()
        self._act = {}
        self.smoothed = bool((o["smooth_scale"].float() != 1).any())     # (an all-ones vector: no division needed)

    def forward(self, x, residual=None, swiglu=False):
        """residual (row shards, bf16 [M, N], no bias): added to the layer's output — inside rank 0's launch, so that
        the all-reduce carries it. swiglu (local_scale only): x is [M, 2 K_local] = [gate | up] of this rank's columns
        and the layer's input is silu(gate) * up, formed inside the quantiser launch."""
        from . import fp4
        o = self.ops
        x = x.to(torch.bfloat16).contiguous()
        assert not swiglu or self.local_scale
        smooth = o["smooth_scale"] if self.smoothed else None
        gscale = None
        if self.kind == "row" and not self.local_scale:
            gscale = agree_on_activation_scale(x, smooth, group=self.group)
        q = fp4.quantize_activation(x, smooth=smooth, w_gscale=o["w_gscale"], rows=self.M, out=self._act.get(swiglu), gscale=gscale,
                                    swiglu=swiglu)
        self._act[swiglu] = q
        self.gemm.alpha = q["alpha"]
        if residual is not None:
            assert self.kind == "row" and o.get("bias") is None
            rank = dist.get_rank(self.group) if dist.is_initialized() else 0
            self.gemm.residual = residual if rank == 0 else None
        elif o.get("bias") is None:
            self.gemm.residual = None
        red = None
        if (self.kind == "row" and self.peer_allreduce and x.is_cuda and dist.is_initialized() and dist.get_world_size(self.group) > 1
                and dist.get_backend(self.group) == "nccl"):
            red = PeerAllReduce.for_group(self.group, x.device, self.M * self.N)
            # the fused launch's epilogue stores its outputs to the peers itself (tile kernels; the gather follows below)
            self.gemm.peer_push = red.push_args() if (self.epilogue_push and self.gemm.mode != 7) else None
        y = self.gemm(q["A"], q["A_sf"], q["X"], A_rec=q.get("A_rec")).view(-1, self.N)[: self.M]
        if self.kind == "row":
            y = y.contiguous()
            if dist.is_initialized() and dist.get_world_size(self.group) > 1:
                if red is not None:
                    return red(y, pushed=self.gemm.peer_push is not None)      # fp32 partials in, bf16 sum out
                dist.all_reduce(y, op=dist.ReduceOp.SUM, group=self.group)      # fp32 [M, N] over NVLink
            y = y.to(torch.bfloat16)
        return y

    __call__ = forward
