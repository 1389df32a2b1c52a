"""Fused Lion optimizer with the reference's torch.optim interface.

Mirrors fast_ops/lion/lion_optimizer.py of jfc4050/fast-ops (`Lion.__init__` :34-55, `step`
:57-76): same constructor defaults, `RuntimeError` on a non-positive learning rate or a beta
outside [0, 1], state key "exp_avg", param-group keys lr / betas / weight_decay.  Instead of
one kernel launch per tensor, `step()` hands every (param, grad, exp_avg) triple of a group to
ONE multi-tensor kernel launch per dtype combination.  The arithmetic follows the reference
torch implementation (fast_ops/lion/lion_optimizer_ref.py:51-67) rounding for rounding.

Keyword-only extensions:
  momentum_dtype   dtype of exp_avg (default: the parameter's dtype, as the reference does at
                   :68-74; the Lion paper keeps momentum in bf16).
  process_group    a torch.distributed group: parameters are laid out in one flat buffer, each
                   rank updates only its 1/world_size slice (and keeps momentum only for it),
                   then ONE all-gather distributes the updated weights (ZeRO-1).
  fused_gather     with process_group: the flat parameter buffer is a symmetric-memory
                   allocation and the step kernel itself stores the updated slice into every
                   peer's buffer over NVLink, replacing the all-gather.
  reduce_gradients with process_group: step() first averages the flat gradient buffer across
                   the ranks with one reduce-scatter into this rank's slice (otherwise the caller
                   is expected to have reduced the gradients already).
"""
from __future__ import annotations

import ctypes
from typing import Dict, Iterable, List, Optional, Tuple

import torch
from torch import Tensor
from torch.optim.optimizer import Optimizer

from .. import _lib
from .zero1 import FlatLayout


def lion_update(param: Tensor, grad: Tensor, exp_avg: Tensor, lr: float, beta1: float, beta2: float,
                weight_decay: float) -> None:
    """Single-tensor fused step; the signature of the reference extension's `lion_update`
    (fast_ops/lion/lion.cpp:4-15).  Same checks as its host launcher
    (fast_ops/lion/lion_update.cu:132-139): param/grad dtypes equal, all three dense."""
    _check_triple(param, grad, exp_avg)
    lib = _lib.load()
    _lib.check(lib.fo_lion_update(
        param.data_ptr(), grad.data_ptr(), exp_avg.data_ptr(), param.numel(),
        _lib.dtype_code(param.dtype), _lib.dtype_code(grad.dtype), _lib.dtype_code(exp_avg.dtype),
        float(lr), float(beta1), float(beta2), float(weight_decay), param.device.index,
        _lib.current_stream_ptr(param.device)))


def _is_dense(t: Tensor) -> bool:
    """True when the tensor's elements fill one gap-free block of memory in some order
    (the reference's `is_non_overlapping_and_dense`, fast_ops/lion/lion_update.cu:109-112)."""
    if t.is_contiguous() or t.numel() == 0:
        return True
    strides = sorted((st, sz) for st, sz in zip(t.stride(), t.shape) if sz != 1)
    expect = 1
    for st, sz in strides:
        if st != expect:
            return False
        expect *= sz
    return True


def _check_triple(param: Tensor, grad: Tensor, exp_avg: Tensor) -> None:
    if not param.is_cuda:
        raise RuntimeError("fast_ops_b200 Lion needs CUDA tensors (there is no CPU path)")
    if grad.device != param.device or exp_avg.device != param.device:
        raise RuntimeError("param, grad and exp_avg must be on the same device")
    if param.dtype != grad.dtype:
        raise RuntimeError(f"param and grad dtypes differ: {param.dtype} vs {grad.dtype}")
    if grad.shape != param.shape or exp_avg.numel() != param.numel():
        raise RuntimeError("param, grad and exp_avg must have the same number of elements")
    for t in (param, grad, exp_avg):
        if not _is_dense(t):
            raise RuntimeError("expected tensor to be contiguous")
    if param.stride() != grad.stride():
        raise RuntimeError("param and grad must share a memory layout")


def _flat_step_push(p: Tensor, g: Tensor, m_shard: Tensor, begin: int, end: int, peer_ptrs, lr: float, betas,
                    wd: float) -> None:
    """Lion step on [begin, end) that also stores the result into the peers' flat buffers
    (C-ABI fo_lion_flat_step_push).  `peer_ptrs`: device addresses of the peers' element 0."""
    lib = _lib.load()
    n = len(peer_ptrs)
    arr = (ctypes.c_void_p * max(n, 1))(*peer_ptrs)
    _lib.check(lib.fo_lion_flat_step_push(
        p.data_ptr(), g.data_ptr(), m_shard.data_ptr(), begin, end, arr, n,
        _lib.dtype_code(p.dtype), _lib.dtype_code(g.dtype), _lib.dtype_code(m_shard.dtype),
        float(lr), float(betas[0]), float(betas[1]), float(wd), p.device.index,
        _lib.current_stream_ptr(p.device)))


def _flat_step(p: Tensor, g: Tensor, m_shard: Tensor, begin: int, end: int, lr: float, betas, wd: float) -> None:
    """Lion step on elements [begin, end) of the flat buffers (C-ABI fo_lion_flat_step)."""
    lib = _lib.load()
    _lib.check(lib.fo_lion_flat_step(
        p.data_ptr(), g.data_ptr(), m_shard.data_ptr(), begin, end,
        _lib.dtype_code(p.dtype), _lib.dtype_code(g.dtype), _lib.dtype_code(m_shard.dtype),
        float(lr), float(betas[0]), float(betas[1]), float(wd), p.device.index,
        _lib.current_stream_ptr(p.device)))


class _TensorList:
    """ctypes image of one multi-tensor call, reused while the pointers stay the same."""

    def __init__(self, key, params: List[Tensor], grads: List[Tensor], moms: List[Tensor]):
        n = len(params)
        self.key = key
        self.n = n
        self.params = (ctypes.c_void_p * n)(*[t.data_ptr() for t in params])
        self.grads = (ctypes.c_void_p * n)(*[t.data_ptr() for t in grads])
        self.moms = (ctypes.c_void_p * n)(*[t.data_ptr() for t in moms])
        self.numels = (ctypes.c_int64 * n)(*[t.numel() for t in params])


class Lion(Optimizer):
    """Lion ("Symbolic Discovery of Optimization Algorithms", arXiv:2302.06675), fused."""

    def __init__(self, params: Iterable, lr: float = 1e-4, betas: Tuple[float, float] = (0.9, 0.99),
                 weight_decay: float = 0.0, *, momentum_dtype: Optional[torch.dtype] = None,
                 process_group=None, fused_gather: bool = False, reduce_gradients: bool = False) -> None:
        if lr <= 0:
            raise RuntimeError(f"expected positive LR, got {lr}")
        if not all(0 <= beta <= 1 for beta in betas):
            raise RuntimeError(f"betas must be between 0 and 1. got {betas}")
        if momentum_dtype not in (None, torch.float16, torch.bfloat16, torch.float32):
            raise RuntimeError(f"unsupported momentum dtype {momentum_dtype}")
        defaults = {"lr": lr, "betas": betas, "weight_decay": weight_decay}
        super().__init__(params, defaults)
        self._momentum_dtype = momentum_dtype
        self._lists: Dict[int, tuple] = {}  # group index -> (address signature, prepared launches)
        self._pg = process_group
        self._zero = None
        if fused_gather and process_group is None:
            raise RuntimeError("fused_gather needs a process_group")
        if reduce_gradients and process_group is None:
            raise RuntimeError("reduce_gradients needs a process_group")
        if process_group is not None:
            self._zero = _Zero1State(self, process_group, momentum_dtype, fused_gather, reduce_gradients)

    # -- multi-tensor path ---------------------------------------------------------------
    @staticmethod
    def _signature(group) -> List[int]:
        """Addresses of every parameter and of its gradient (0 = no gradient), in order: what
        decides whether the launches prepared for this group last step can be issued again."""
        sig = []
        for param in group["params"]:
            grad = param.grad
            sig.append(param.data_ptr())
            sig.append(0 if grad is None else grad.data_ptr())
        return sig

    def _prepare_group(self, gi: int, group) -> list:
        """Checks every (param, grad, exp_avg) triple of the group, creates missing momentum, and
        returns one prepared launch (a `_TensorList`) per (device, dtype, momentum dtype)."""
        buckets: Dict[tuple, Tuple[List[Tensor], List[Tensor], List[Tensor]]] = {}
        for param in group["params"]:
            grad = param.grad
            if grad is None:
                continue
            state = self.state[param]
            if "exp_avg" not in state:
                state["exp_avg"] = torch.zeros_like(
                    param, dtype=self._momentum_dtype or param.dtype, memory_format=torch.preserve_format)
            exp_avg = state["exp_avg"]
            _check_triple(param, grad, exp_avg)
            key = (gi, param.device.index, param.dtype, exp_avg.dtype)
            ps, gs, ms = buckets.setdefault(key, ([], [], []))
            ps.append(param)
            gs.append(grad)
            ms.append(exp_avg)
        return [_TensorList(key, ps, gs, ms) for key, (ps, gs, ms) in buckets.items()]

    @torch.no_grad()
    def step(self) -> None:
        """Parameter and momentum update (no closure, no return value: lion_optimizer.py:57)."""
        if self._zero is not None:
            self._zero.step()
            return
        lib = _lib.load()
        for gi, group in enumerate(self.param_groups):
            # A training loop presents the same tensors step after step: while no parameter or
            # gradient address has changed, the checks and the pointer arrays of the last step stand.
            sig = self._signature(group)
            cached = self._lists.get(gi)
            if cached is None or cached[0] != sig:
                cached = (sig, self._prepare_group(gi, group))
                self._lists[gi] = cached
            lr = float(group["lr"])
            weight_decay = float(group["weight_decay"])
            beta1, beta2 = (float(b) for b in group["betas"])
            for tl in cached[1]:
                _, device_index, p_dtype, m_dtype = tl.key
                _lib.check(lib.fo_lion_multi_tensor_step(
                    tl.params, tl.grads, tl.moms, tl.numels, tl.n,
                    _lib.dtype_code(p_dtype), _lib.dtype_code(p_dtype), _lib.dtype_code(m_dtype),
                    lr, beta1, beta2, weight_decay, device_index,
                    _lib.current_stream_ptr(torch.device("cuda", device_index))))

    def load_state_dict(self, state_dict) -> None:
        """As torch.optim.Optimizer.load_state_dict; in process_group mode the loaded momentum
        (this rank's slices, as state_dict() saved them) is copied back into the rank's shard."""
        super().load_state_dict(state_dict)
        self._lists.clear()  # the momentum tensors are new objects
        if self._zero is not None:
            self._zero.adopt_loaded_state()

    # -- ZeRO-1 accessors ------------------------------------------------------------------
    @property
    def flat_params(self) -> Optional[Tensor]:
        return None if self._zero is None else self._zero.flat_p

    @property
    def flat_grads(self) -> Optional[Tensor]:
        return None if self._zero is None else self._zero.flat_g


class _Zero1State:
    """Flat parameter / gradient buffers, this rank's momentum shard and the step that uses them.

    Every parameter becomes a view into `flat_p`; `p.grad` is pre-set to a view into `flat_g`
    so that backward accumulates straight into it (a caller that assigns other gradient
    tensors pays one copy per tensor in step()).  Gradient averaging across ranks is the
    caller's job (reduce-scatter or all-reduce before step()); the optimizer's one collective is
    the all-gather of updated weights.
    """

    def __init__(self, opt: Lion, group, momentum_dtype: Optional[torch.dtype], fused_gather: bool = False,
                 reduce_gradients: bool = False):
        import torch.distributed as dist

        self.reduce_gradients = reduce_gradients
        self.opt = opt
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        params = [p for g in opt.param_groups for p in g["params"]]
        if not params:
            raise RuntimeError("no parameters")
        if len(opt.param_groups) != 1:
            raise RuntimeError("process_group mode supports a single param group")
        dtype, device = params[0].dtype, params[0].device
        for p in params:
            if p.dtype != dtype or p.device != device:
                raise RuntimeError("process_group mode needs all parameters on one device with one dtype")
        self.params = params
        self.layout = FlatLayout.build([p.numel() for p in params], self.world)
        self.symm = None
        self.peer_ptrs: List[int] = []
        if fused_gather and self.world > 1:
            # peer-mapped allocation: every rank can store into every other rank's buffer
            import torch.distributed._symmetric_memory as symm_mem

            self.flat_p = symm_mem.empty(self.layout.total, dtype=dtype, device=device)
            self.flat_p.zero_()
            self.symm = symm_mem.rendezvous(self.flat_p, group)
            ptrs = list(self.symm.buffer_ptrs)
            self.peer_ptrs = [int(ptrs[r]) for r in range(self.world) if r != self.rank]
        else:
            self.flat_p = torch.zeros(self.layout.total, dtype=dtype, device=device)
        self.flat_g = torch.zeros(self.layout.total, dtype=dtype, device=device)
        self._grad_views: List[Tensor] = []
        with torch.no_grad():
            for p, off in zip(params, self.layout.offsets):
                n = p.numel()
                view = self.flat_p[off:off + n].view(p.shape)
                view.copy_(p.data.contiguous())
                p.data = view
                gview = self.flat_g[off:off + n].view(p.shape)
                if p.grad is not None:
                    gview.copy_(p.grad)
                p.grad = gview
                self._grad_views.append(gview)
        self.begin, self.end = self.layout.shard_range(self.rank)
        self.m_shard = torch.zeros(self.end - self.begin, dtype=momentum_dtype or dtype, device=device)
        for i, p in enumerate(params):
            _, s0, n = self.layout.tensor_slice_in_shard(i, self.rank)
            opt.state[p]["exp_avg"] = self.m_shard[s0:s0 + n]
        self.flat_step_fn = _flat_step

    def adopt_loaded_state(self) -> None:
        """After Optimizer.load_state_dict: state[p]["exp_avg"] holds fresh tensors; copy them
        into the shard and point the state back at views of it."""
        with torch.no_grad():
            for i, p in enumerate(self.params):
                _, s0, n = self.layout.tensor_slice_in_shard(i, self.rank)
                view = self.m_shard[s0:s0 + n]
                loaded = self.opt.state[p].get("exp_avg")
                if loaded is not None and loaded.data_ptr() != view.data_ptr():
                    if loaded.numel() != n:
                        raise RuntimeError("loaded exp_avg does not match this rank's slice of the parameter")
                    view.copy_(loaded.reshape(-1))
                self.opt.state[p]["exp_avg"] = view

    def _average_gradients(self) -> None:
        import torch.distributed as dist

        shard = self.flat_g[self.begin:self.end]
        if dist.get_backend(self.group) == "gloo":  # no reduce-scatter there: all-reduce, keep the slice
            dist.all_reduce(self.flat_g, group=self.group)
            shard.div_(self.world)
        else:
            dist.reduce_scatter_tensor(shard, self.flat_g, op=dist.ReduceOp.AVG, group=self.group)

    @torch.no_grad()
    def step(self) -> None:
        import torch.distributed as dist

        for p, gview in zip(self.params, self._grad_views):
            if p.grad is None:
                raise RuntimeError("process_group mode needs a gradient for every parameter")
            if p.grad.data_ptr() != gview.data_ptr():
                gview.copy_(p.grad)
                p.grad = gview
        if self.reduce_gradients and self.world > 1:
            self._average_gradients()
        group = self.opt.param_groups[0]
        if self.symm is not None:
            # ranks meet before any of them overwrites a peer's weights, and again before any of
            # them reads the gathered result (device-side barriers on the current stream)
            self.symm.barrier(channel=0)
            _flat_step_push(self.flat_p, self.flat_g, self.m_shard, self.begin, self.end, self.peer_ptrs,
                            group["lr"], group["betas"], group["weight_decay"])
            self.symm.barrier(channel=1)
            return
        self.flat_step_fn(self.flat_p, self.flat_g, self.m_shard, self.begin, self.end, group["lr"],
                          group["betas"], group["weight_decay"])
        if self.world > 1:
            dist.all_gather_into_tensor(self.flat_p, self.flat_p[self.begin:self.end], group=self.group)
