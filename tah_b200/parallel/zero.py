"""ZeRO-style data parallelism: sharded fp32 master weights + AdamW, full bf16 params and grads.

The reference trains through HuggingFace ``Trainer`` + DeepSpeed ZeRO-2/3 configured in YAML
(reference ``script/recipes/accelerate_configs/zero2.yaml``); nothing of it is in-tree.  Here
the optimizer is part of the framework:

* all trainable parameters live in ONE flat bf16 buffer and their gradients in another, both in
  symmetric memory on CUDA, with the parameters / ``.grad`` of the model being views into them;
* each rank owns the fp32 master copy and Adam moments of a contiguous 1/world shard;
* ``step()`` = gradient reduce-scatter fused with scaling and the squared-norm partial sum, a scalar
  all-reduce for global-norm clipping, then AdamW fused with the parameter broadcast
  (``csrc/optim.cu``; NVLS multimem when available, peer loads/stores otherwise).

On CPU (gloo) the same class runs a PyTorch statement of the algorithm (all-reduce, shard update,
all-gather), which is what the multi-process CPU tests exercise; the two paths compute the same
update.  ``world_size == 1`` degenerates to a fused single-GPU AdamW with fp32 master weights.
"""
from __future__ import annotations

import math
from typing import Iterable, List, Optional

import torch
import torch.distributed as dist

MAX_GRID = 148


class ZeroAdamW:
    def __init__(self, params: Iterable[torch.nn.Parameter], group=None, lr: float = 1e-4, betas=(0.9, 0.999),
                 eps: float = 1e-8, weight_decay: float = 0.01, max_grad_norm: float = 0.0,
                 use_multicast: bool = True, no_decay: Optional[Iterable[torch.nn.Parameter]] = None):
        """``no_decay``: parameters that take no weight decay (norm gains, biases, thresholds; the HuggingFace
        trainer the reference builds on excludes LayerNorm and bias parameters from decay).  They are laid out
        behind the decayed ones in the flat buffers, so the kernel needs one boundary index."""
        skip = {id(p) for p in (no_decay or [])}
        ps = [p for p in params if p.requires_grad]
        self.params: List[torch.nn.Parameter] = [p for p in ps if id(p) not in skip] + [p for p in ps if id(p) in skip]
        self.decay_numel = sum(p.numel() for p in ps if id(p) not in skip)
        if not self.params:
            raise ValueError("no trainable parameters")
        self.group = group
        self.dist_on = dist.is_available() and dist.is_initialized() and (group is not None or dist.get_world_size() > 1)
        self.world = dist.get_world_size(group) if self.dist_on else 1
        self.rank = dist.get_rank(group) if self.dist_on else 0
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.max_grad_norm = max_grad_norm
        self.step_count = 0
        self.device = self.params[0].device
        self.dtype = self.params[0].dtype
        if any(p.dtype != self.dtype or p.device != self.device for p in self.params):
            raise ValueError("ZeroAdamW needs all trainable parameters on one device with one dtype")
        self.cuda = self.device.type == "cuda" and self.dtype == torch.bfloat16
        n = sum(p.numel() for p in self.params)
        align = 8 * self.world
        self.numel = n
        self.padded = (n + align - 1) // align * align
        self.shard = self.padded // self.world
        self.lo, self.hi = self.rank * self.shard, (self.rank + 1) * self.shard
        self._alloc_flat(use_multicast)
        # move parameters and gradients into the flat buffers (views)
        off = 0
        with torch.no_grad():
            for p in self.params:
                k = p.numel()
                self.flat_param[off:off + k].copy_(p.detach().reshape(-1))
                p.data = self.flat_param[off:off + k].view_as(p)
                p.grad = self.flat_grad[off:off + k].view_as(p)
                off += k
        self.flat_grad.zero_()
        if self.dist_on and self.world > 1:
            # every rank starts from rank 0's values, whatever its local initialisation seed was
            dist.broadcast(self.flat_param, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        self.master = self.flat_param[self.lo:self.hi].float().clone()
        self.m = torch.zeros_like(self.master)
        self.v = torch.zeros_like(self.master)
        self.gshard = torch.zeros_like(self.master)
        self.norm_sq = torch.zeros(1, dtype=torch.float32, device=self.device)
        self.last_grad_norm: Optional[torch.Tensor] = None

    # ------------------------------------------------------------------------------------------
    def _alloc_flat(self, use_multicast: bool) -> None:
        self.mc_grad = self.mc_param = 0
        if self.cuda and self.world > 1:
            import torch.distributed._symmetric_memory as symm_mem
            g = self.group if self.group is not None else dist.group.WORLD
            mk = lambda n, dt: symm_mem.empty(n, dtype=dt, device=self.device)
            self.flat_param = mk(self.padded, self.dtype)
            self.flat_grad = mk(self.padded, self.dtype)
            self._flags = mk(MAX_GRID * self.world, torch.int32)
            self.flat_param.zero_()
            self.flat_grad.zero_()
            self._flags.zero_()
            hp, hg, hf = (symm_mem.rendezvous(t, g) for t in (self.flat_param, self.flat_grad, self._flags))
            self._handles = (hp, hg, hf)
            self.param_ptrs = [int(x) for x in hp.buffer_ptrs]
            self.grad_ptrs = [int(x) for x in hg.buffer_ptrs]
            self.flag_ptrs = [int(x) for x in hf.buffer_ptrs]
            if use_multicast:
                mp, mg = int(getattr(hp, "multicast_ptr", 0) or 0), int(getattr(hg, "multicast_ptr", 0) or 0)
                if mp and mg:
                    self.mc_param, self.mc_grad = mp, mg
            self.epoch = torch.zeros(MAX_GRID, dtype=torch.int32, device=self.device)
            torch.cuda.synchronize(self.device)
            dist.barrier(g)
        else:
            self.flat_param = torch.zeros(self.padded, dtype=self.dtype, device=self.device)
            self.flat_grad = torch.zeros(self.padded, dtype=self.dtype, device=self.device)
            if self.cuda:
                self._flags = torch.zeros(MAX_GRID, dtype=torch.int32, device=self.device)
                self.epoch = torch.zeros(MAX_GRID, dtype=torch.int32, device=self.device)
                self.param_ptrs = [self.flat_param.data_ptr()]
                self.grad_ptrs = [self.flat_grad.data_ptr()]
                self.flag_ptrs = [self._flags.data_ptr()]

    # ------------------------------------------------------------------------------------------
    def zero_grad(self, set_to_none: bool = False) -> None:
        self.flat_grad.zero_()
        off = 0
        for p in self.params:       # autograd may have replaced .grad; point it back at the flat buffer
            k = p.numel()
            want = self.flat_grad[off:off + k].view_as(p)
            if p.grad is None or p.grad.data_ptr() != want.data_ptr():
                p.grad = want
            off += k

    def _collect_stray_grads(self) -> None:
        off = 0
        for p in self.params:
            k = p.numel()
            view = self.flat_grad[off:off + k].view_as(p)
            if p.grad is not None and p.grad.data_ptr() != view.data_ptr():
                view.add_(p.grad.to(view.dtype))
                p.grad = view
            off += k

    @torch.no_grad()
    def accumulate(self) -> None:
        """Fold the gradient of the micro-batch that just finished its backward into an fp32 accumulator and clear
        the 16-bit gradient buffer.  Call after every backward of an accumulation window: the sum over the window is
        then rounded to the parameter dtype once (at :meth:`step`) instead of after every micro-batch (what
        DeepSpeed's bf16 optimizer does with ``grad_accum_dtype: fp32``; the reference trains with 16 accumulation
        steps, ``script/recipes/qwen3_1.7/sft_tah_step1.yaml:46-47``).  Costs 4 bytes per trainable parameter."""
        self._collect_stray_grads()
        if self.flat_grad.dtype == torch.float32:
            return                                        # fp32 parameters accumulate in fp32 already
        if getattr(self, "acc32", None) is None:
            self.acc32 = torch.zeros(self.padded, dtype=torch.float32, device=self.device)
        self.acc32.add_(self.flat_grad)
        self.flat_grad.zero_()
        self._acc_pending = True

    def _flush_accumulator(self) -> None:
        if getattr(self, "_acc_pending", False):
            self.acc32.add_(self.flat_grad)               # a backward since the last accumulate() call, if any
            self.flat_grad.copy_(self.acc32)
            self.acc32.zero_()
            self._acc_pending = False

    @torch.no_grad()
    def step(self, grad_scale: float = 1.0, lr: Optional[float] = None,
             extra_norm_sq: Optional[torch.Tensor] = None, norm_hook=None) -> torch.Tensor:
        """One update.  ``grad_scale`` multiplies the rank-averaged gradient (e.g. 1 for losses already
        normalised over the accumulation window).  ``extra_norm_sq`` (optional device scalar): this rank's
        share of the squared gradient norm of parameters managed elsewhere (parameter-sharded units); it joins
        the all-reduce, so clipping uses the norm over both sets.  ``norm_hook(self)`` (optional) is called once
        the rank-averaged, scaled gradient shard is in ``self.gshard`` (flat elements ``[self.lo, self.hi)``) and
        returns a further share of the squared norm (tensor-parallel training adds the other ranks' shards there).
        Returns the global gradient norm (device tensor); ``self.norm_sq`` holds its square."""
        self._collect_stray_grads()
        self._flush_accumulator()
        self.step_count += 1
        lr = self.lr if lr is None else lr
        b1, b2 = self.betas
        bc1, bc2 = 1.0 - b1 ** self.step_count, 1.0 - b2 ** self.step_count
        scale = grad_scale / self.world
        if self.cuda:
            return self._step_cuda(scale, lr, b1, b2, bc1, bc2, extra_norm_sq, norm_hook)
        return self._step_torch(scale, lr, b1, b2, bc1, bc2, extra_norm_sq, norm_hook)

    # ---- CUDA: fused kernels over peer memory -------------------------------------------------
    def _step_cuda(self, scale, lr, b1, b2, bc1, bc2, extra_norm_sq=None, norm_hook=None):
        import ctypes
        from tah_b200.ops import cuda as K
        lib = K.lib()
        n = len(self.grad_ptrs)
        arr = lambda ptrs: (ctypes.c_void_p * n)(*ptrs)
        cf, ci, cll, cvp = ctypes.c_float, ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p
        stream = cvp(torch.cuda.current_stream().cuda_stream)
        grid = max(1, min(MAX_GRID, (self.shard // 8 + 255) // 256))
        self.norm_sq.zero_()

        def launch(phase):
            if phase == 1:
                lib.tahb_zero_set_nodecay_from(cll(self.decay_numel))
            rc = lib.tahb_zero_step(ci(phase), arr(self.grad_ptrs), arr(self.param_ptrs), cvp(self.mc_grad),
                                    cvp(self.mc_param), cvp(self.gshard.data_ptr()), cvp(self.master.data_ptr()),
                                    cvp(self.m.data_ptr()), cvp(self.v.data_ptr()), cvp(self.norm_sq.data_ptr()),
                                    arr(self.flag_ptrs), cvp(self.epoch.data_ptr()),
                                    cvp(K.status_word(self.device).data_ptr()), cll(self.lo), cll(self.hi),
                                    ci(self.rank), ci(self.world), cf(scale), cf(lr), cf(b1), cf(b2), cf(self.eps),
                                    cf(self.weight_decay), cf(bc1), cf(bc2), cf(self.max_grad_norm), ci(grid), stream)
            if rc != 0:
                raise RuntimeError(f"tahb_zero_step phase {phase} failed (code {rc})")

        launch(0)
        if extra_norm_sq is not None:
            self.norm_sq += extra_norm_sq.to(self.norm_sq.dtype)
        if norm_hook is not None:
            self.norm_sq += norm_hook(self).to(self.norm_sq.dtype).reshape(1)
        if self.world > 1:
            dist.all_reduce(self.norm_sq, group=self.group)
        launch(1)
        self.last_grad_norm = self.norm_sq.sqrt()
        return self.last_grad_norm

    # ---- CPU / generic: PyTorch statement of the same algorithm --------------------------------
    def _step_torch(self, scale, lr, b1, b2, bc1, bc2, extra_norm_sq=None, norm_hook=None):
        g_full = self.flat_grad.float()
        if self.world > 1:
            dist.all_reduce(g_full, group=self.group)
        g = g_full[self.lo:self.hi] * scale
        nsq = (g * g).sum().reshape(1)
        if extra_norm_sq is not None:
            nsq = nsq + extra_norm_sq.to(nsq.dtype).reshape(1)
        if norm_hook is not None:
            self.gshard = g
            nsq = nsq + norm_hook(self).to(nsq.dtype).reshape(1)
        if self.world > 1:
            dist.all_reduce(nsq, group=self.group)
        self.norm_sq = nsq
        norm = nsq.sqrt()
        if self.max_grad_norm > 0:
            g = g * torch.clamp(self.max_grad_norm / (norm + 1e-6), max=1.0)
        self.m.mul_(b1).add_(g, alpha=1 - b1)
        self.v.mul_(b2).addcmul_(g, g, value=1 - b2)
        upd = (self.m / bc1) / ((self.v / bc2).sqrt() + self.eps)
        decay = (torch.arange(self.lo, self.hi, device=self.master.device) < self.decay_numel).to(self.master.dtype)
        self.master.mul_(1 - lr * self.weight_decay * decay).add_(upd, alpha=-lr)
        new = self.master.to(self.dtype)
        if self.world > 1:
            parts = [torch.empty_like(new) for _ in range(self.world)]
            dist.all_gather(parts, new, group=self.group)
            self.flat_param.copy_(torch.cat(parts))
        else:
            self.flat_param[self.lo:self.hi].copy_(new)
        self.last_grad_norm = norm[0]
        return self.last_grad_norm

    # ---- state ---------------------------------------------------------------------------------
    def state_dict(self) -> dict:
        return {"step": self.step_count, "master": self.master.cpu(), "m": self.m.cpu(), "v": self.v.cpu(),
                "rank": self.rank, "world": self.world, "lo": self.lo, "hi": self.hi, "numel": self.numel}

    def load_state_dict(self, sd: dict) -> None:
        if sd["world"] != self.world or sd["lo"] != self.lo or sd["hi"] != self.hi:
            raise ValueError("optimizer shard layout differs from the checkpoint (world size changed?)")
        self.step_count = int(sd["step"])
        for name in ("master", "m", "v"):
            getattr(self, name).copy_(sd[name].to(self.device))
        self.flat_param[self.lo:self.hi].copy_(self.master.to(self.dtype))
