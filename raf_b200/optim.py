"""Python mirror of ``raf.optim`` for the optimizer-step path: the eager optimizers
(``python/raf/optim/sgd.py:21-58``, ``python/raf/optim/lans.py:22-104``) and the ZeRO-aware
wrappers ``with_sgd`` / ``with_lans`` (``sgd.py:61-230``, ``lans.py:107-330``), on torch CUDA
tensors.  Constructor arguments, defaults, state names (``sgd.{i}.v``, ``{name}.sgd_w``,
``{name}.lans_w``, ``{name}.m`` ...) and error behaviour follow the reference; the arithmetic
runs in the CUDA kernels behind :mod:`raf_b200.op` and :mod:`raf_b200.zero`.

The reference's wrappers trace a model's forward/backward and append the update to the
graph; here the wrapper owns only what comes after backward: it takes the gradients and runs
reduce-scatter -> update -> all-gather.
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Optional, Sequence

import torch

from . import distributed as dist
from . import op
from .zero import Plan, ZeroStep, make_hyper


class SGD:
    """``raf.optim.SGD(params, learning_rate, momentum=0)``: x.grad is read, x and the momentum
    buffer ``sgd.{i}.v`` are updated with one ``raf.op.sgd`` per parameter."""

    def __init__(self, params: Iterable[torch.Tensor], learning_rate, momentum=0):
        if learning_rate < 0.0:
            raise ValueError("Invalid learning rate: {}".format(learning_rate))
        if momentum < 0.0:
            raise ValueError("Invalid momentum value: {}".format(momentum))
        self.params = []
        self._lr = learning_rate
        self._momentum = momentum
        for x in params:
            assert isinstance(x, torch.Tensor) and x.is_cuda, "Only CUDA tensors can be optimized!"
            self.params.append((x, torch.zeros_like(x, dtype=torch.float32)))

    def state(self) -> Dict[str, torch.Tensor]:
        return {f"sgd.{i}.v": v for i, (_, v) in enumerate(self.params)}

    def step(self):
        """Update the parameters with gradients."""
        for x0, v0 in self.params:
            if x0.grad is None:
                continue
            op.sgd_(x0.data, x0.grad, v0, self._lr, self._momentum)


class LANS:
    """``raf.optim.LANS``: one ``raf.op.lans`` call over every parameter that has a gradient;
    the step counter starts at 1 (``lans.py:66``)."""

    def __init__(self, params: Iterable[torch.Tensor], lr=1e-3, betas=(0.9, 0.999), eps=1e-6,
                 weight_decay=0.01, bias_correction=True, grad_averaging=True, mode=True,
                 normalize_grad=True):
        self.lr = lr
        self.beta1, self.beta2 = betas
        self.eps = eps
        self.weight_decay = weight_decay
        self.bias_correction = bias_correction
        self.grad_averaging = grad_averaging
        self.mode = mode
        self.normalize_grad = normalize_grad
        self.params = []
        self._step = 1
        for x in params:
            assert isinstance(x, torch.Tensor) and x.is_cuda, "Only CUDA tensors can be optimized!"
            self.params.append((x, torch.zeros_like(x, dtype=torch.float32),
                                torch.zeros_like(x, dtype=torch.float32)))

    def state(self) -> Dict[str, torch.Tensor]:
        out = {}
        for i, (_, m, v) in enumerate(self.params):
            out[f"lans.{i}.m"] = m
            out[f"lans.{i}.v"] = v
        return out

    def step(self):
        """Update the parameters with gradients."""
        g_list, x_list, m_list, v_list = [], [], [], []
        for x, m, v in self.params:
            if x.grad is None:
                continue
            g_list.append(x.grad)
            x_list.append(x.data)
            m_list.append(m)
            v_list.append(v)
        if x_list:
            op.lans(g_list + x_list + m_list + v_list, self._step, self.lr, self.beta1, self.beta2,
                    self.eps, int(self.bias_correction), self.weight_decay, int(self.grad_averaging),
                    int(self.mode), bool(self.normalize_grad))
        self._step += 1


class _ZeroWrapper:
    """State and step shared by :func:`with_sgd` and :func:`with_lans`."""

    def __init__(self, model_state: Dict[str, torch.Tensor], optimizer: str, prefix: str,
                 hyper_kwargs: dict, grad_dtype=None):
        dcfg, comm = dist.get_config(), dist.get_communicator()
        self.names = list(model_state)
        self.model_params = [model_state[n] for n in self.names]
        for p in self.model_params:
            assert p.is_cuda and p.is_contiguous(), "parameters must be compact CUDA tensors"
        self.dtype = self.model_params[0].dtype  # model dtype: that of the first parameter
        self.optimizer, self.prefix = optimizer, prefix
        self.zero_opt_level = dcfg.zero_opt_level
        n = comm.size if dcfg.zero_opt_level else 1
        rank = comm.rank if dcfg.zero_opt_level else 0
        # zero_opt_level 0 on several ranks: plain data parallelism - every rank keeps the whole
        # state, the gradients are averaged in place by _allreduce (what AutoDataParallel inserts,
        # src/pass/data_parallel.cc) and the update runs unsharded
        self._allreduce_first = n != comm.size
        if self._allreduce_first:
            comm = self._local_comm = dist.Communicator(1, 0, torch.cuda.current_device())
        self.plan = Plan([tuple(p.shape) for p in self.model_params], n, rank,
                         int(dcfg.group_bucket_size))
        gdt = grad_dtype if grad_dtype is not None else self.dtype
        self.zero = ZeroStep(self.plan, comm, gdt, self.dtype, optimizer)
        self.state: Dict[str, torch.Tensor] = {}
        self._w, self._m, self._v = [], [], []
        for i, (name, p) in enumerate(zip(self.names, self.model_params)):
            # the fp32 master copy of this rank's row block, zero-padded (split_ndarray_with_padding)
            se = int(self.plan.shard_elems[i])
            padded = torch.zeros(se * n, dtype=torch.float32, device=p.device)
            padded[:p.numel()] = p.detach().reshape(-1).to(torch.float32)
            w = padded[rank * se:(rank + 1) * se].clone()
            m = torch.zeros(se, dtype=torch.float32, device=p.device)
            self._w.append(w)
            self._m.append(m)
            self.state[f"{name}.{prefix}_w"] = w
            if optimizer == "sgd":
                self.state[f"{name}.{prefix}_v"] = m
            else:
                v = torch.zeros(se, dtype=torch.float32, device=p.device)
                self._v.append(v)
                self.state[f"{name}.m"] = m
                self.state[f"{name}.v"] = v
        self.hyper = make_hyper(optimizer, average=1, **hyper_kwargs)
        self.step_no = 0
        self._bound = None

    def step(self, grads: Sequence[torch.Tensor]):
        """One optimizer step from this rank's local gradients (same order as the parameters)."""
        assert len(grads) == len(self.model_params)
        key = tuple(g.data_ptr() for g in grads)
        if key != self._bound:
            self.zero.bind([g.reshape(-1) for g in grads], [p.data.reshape(-1) for p in self.model_params],
                           self._w, self._m, self._v if self.optimizer != "sgd" else None)
            self._bound = key
        self.step_no += 1
        if self._allreduce_first:
            dist.allreduce(list(grads), "avg")
        self.zero.step(self.hyper, self.step_no)

    def close(self):
        self.zero.close()
        self.plan.close()
        if getattr(self, "_local_comm", None) is not None:
            self._local_comm.close()
            self._local_comm = None


def with_sgd(learning_rate=0.1, momentum=0.01):
    """``raf.optim.sgd.with_sgd``: returns a wrapper factory; the wrapper keeps ``{name}.sgd_w``
    (fp32 master shard) and ``{name}.sgd_v`` per parameter."""

    def decorator(model_state: Dict[str, torch.Tensor], grad_dtype=None):
        return _ZeroWrapper(model_state, "sgd", "sgd",
                            dict(learning_rate=learning_rate, mu=momentum), grad_dtype)

    return decorator


def with_lans(lr=1e-3, betas=(0.9, 0.999), eps=1e-6, weight_decay=0.01, bias_correction=True,
              grad_averaging=True, mode=True, normalize_grad=True):
    """``raf.optim.lans.with_lans``: the wrapper keeps ``{name}.lans_w``, ``{name}.m``, ``{name}.v``."""

    def decorator(model_state: Dict[str, torch.Tensor], grad_dtype=None, grad_scale=1.0):
        return _ZeroWrapper(model_state, "lans", "lans",
                            dict(learning_rate=lr, beta1=betas[0], beta2=betas[1], eps=eps,
                                 weight_decay=weight_decay, bias_correction=int(bias_correction),
                                 grad_averaging=int(grad_averaging), mode=int(mode),
                                 normalize_grad=int(normalize_grad), grad_scale=grad_scale),
                            grad_dtype)

    return decorator
