"""A linear layer ``y = act(x W^T + b) (+ residual)`` as parts use it.

The weight is held as ``[out, in]`` with the input dimension contiguous (the
layout the kernels read); a file that stores ``[in, out]`` (HF's Conv1D, as
GPT-2 checkpoints do, which mlx-lm transposes in ``Model.sanitize``,
mlx_lm/models/gpt2.py:175-190) is transposed once at bind time.  Bias, the
activation and the residual add run in the kernel's epilogue.
"""

from __future__ import annotations

from types import SimpleNamespace
from typing import List, Optional

import torch

from .. import ops
from .base import MATRIX, VECTOR, Init, Normed, ParamSpec, Part

# name -> epilogue code, read from the list the kernels are compiled from (csrc/activations.cuh)
ACTIVATIONS = {None: ops.EPI_NONE, **ops.ACTIVATION_CODES}


class Linear(Part):
    replayable = True
    kernel_libs = ("gemm_simt", "gemm_smallm", "gemm_smallm_fold", "gemm_tcgen05")

    def __init__(self, name: str, n_in: int, n_out: int, bias: bool = True, stored: str = "out_in",
                 weight_suffix: str = ".weight", init: Init = Init(), bias_init: Init = Init(),
                 tensor_core_from: Optional[int] = None):
        if stored not in ("out_in", "in_out"):
            raise ValueError(f"stored layout {stored!r}: 'out_in' or 'in_out'")
        self.name, self.n_in, self.n_out, self.has_bias, self.stored = name, n_in, n_out, bias, stored
        self.weight_name = name + weight_suffix
        self.init, self.bias_init = init, bias_init
        self.tensor_core_from = self.TENSOR_CORE_FROM if tensor_core_from is None else int(tensor_core_from)
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None
        self.folded = None        # see fold_norm

    def param_specs(self) -> List[ParamSpec]:
        shape = (self.n_out, self.n_in) if self.stored == "out_in" else (self.n_in, self.n_out)
        specs = [ParamSpec(self.weight_name, shape, MATRIX, self.init)]
        if self.has_bias:
            specs.append(ParamSpec(self.name + ".bias", (self.n_out,), VECTOR, self.bias_init))
        return specs

    def bind(self, tensors, dtype, device) -> None:
        w = tensors[self.weight_name]
        if self.stored == "in_out":
            w = w.t().contiguous()
        self.weight = w
        self.bias = tensors[self.name + ".bias"] if self.has_bias else None

    def use_weight(self, weight: torch.Tensor) -> None:
        """Share another part's ``[out, in]`` tensor (a tied output head)."""
        self.weight = weight

    def fold_norm(self, norm) -> bool:
        """Fold the LayerNorm that feeds this layer into its weights:
        ``LayerNorm(x) W^T + b = rstd (x W'^T - mean colsum) + b'`` with ``W' = W diag(gain)`` (rounded to
        bfloat16 once, here), ``colsum = W' 1`` and ``b' = b + W norm_bias``.  The layer then takes the rows
        before the norm (a ``Normed``): the products run on them as they are and the epilogue applies mean and
        1/std, which the few-rows kernel finds from the fragments it loads anyway (csrc/gemm_smallm.cuh) and
        which for more rows come from a statistics kernel (``ops.row_stats``).  ``W'`` replaces ``W``: every
        step, of few rows or many, goes through the same weights and the same arithmetic."""
        args = norm.fold_args()
        w = self.weight
        if args is None or w is None or w.dtype != torch.bfloat16 or self.n_in % 8 or self.folded is not None:
            return False
        gain, nbias, eps = args
        w32 = w.float()
        folded = (w32 * gain.float()[None, :]).to(torch.bfloat16)
        bias = self.bias.float().clone() if self.bias is not None else torch.zeros(self.n_out, device=w.device)
        if nbias is not None:
            bias += w32 @ nbias.float()
        self.folded = SimpleNamespace(norm=norm, colsum=folded.float().sum(dim=1).contiguous(), eps=float(eps))
        self.weight, self.bias = folded, bias.contiguous()
        return True

    # From this many output features on, steps of 33 to 64 rows run on the tcgen05 kernel rather than on the
    # few-rows kernel (measured with a vocabulary-sized output: each of the few-rows kernel's many CTAs reads
    # all the rows again).  An option of the layer, not of a model: ``Linear(..., tensor_core_from=n)``.
    TENSOR_CORE_FROM = 16384

    def few_rows(self, n_rows: int) -> bool:
        """Whether a step of ``n_rows`` rows runs on the few-rows kernel (else: the tcgen05 kernel)."""
        if n_rows > ops.SMALL_M:
            return False
        return not (n_rows > 32 and self.n_out >= self.tensor_core_from)

    def fold_of(self, ctx, x: Normed, few: Optional[bool] = None):
        """The ``fold`` argument of the kernels for this step's rows: ``(colsum, eps)`` for the few-rows
        kernel, which finds the rows' statistics itself, ``(colsum, stats)`` with the statistics from
        ``ops.row_stats`` for the tcgen05 kernel.  ``few``: which of the two runs (default: ``few_rows``)."""
        f, src = self.folded, x.source
        if (f is None or f.norm is not x.norm or x.rows is not None or src.stride(1) != 1 or src.stride(0) % 8
                or src.data_ptr() % 16):
            raise ops.KernelError(f"{self.name}: the norm before this layer is folded into its weights; it takes "
                                  f"the rows before that norm, contiguous and 16-byte aligned")
        if self.few_rows(x.shape[0]) if few is None else few:
            return (f.colsum, f.eps)
        stats = ctx.ws.get("row_stats", x.shape[0], 2, torch.float32)
        ops.label(f.norm.name + ".statistics", 3.0 * src.shape[0] * src.shape[1], 2.0 * src.shape[0] * src.shape[1])
        ops.row_stats(src, stats, f.eps, ctx.stream)
        return (f.colsum, stats)

    def forward(self, ctx, x, out, activation=None, residual=None) -> torch.Tensor:
        """float32: the generic kernel (true 32-bit arithmetic).  bfloat16: the weight-streaming kernel for up
        to 64 rows, the tcgen05 kernel for more; an inner size that is no multiple of 8 (no 16-byte rows)
        goes to the generic kernel."""
        epi = ACTIVATIONS[activation]
        M = x.shape[0]
        few = self.few_rows(x.shape[0])      # decided once, before the fold's argument is made for that kernel
        fold = None
        if isinstance(x, Normed):
            fold = self.fold_of(ctx, x, few)
            x = x.source
        elif self.folded is not None:
            raise ops.KernelError(f"{self.name}: the norm before this layer is folded into its weights; it takes a "
                                  f"Normed, not a tensor")
        fast = (x.dtype == torch.bfloat16 and self.n_in % 8 == 0 and x.stride(0) % 8 == 0
                and x.data_ptr() % 16 == 0)
        ops.label(self.name, 2.0 * M * self.n_in * self.n_out,
                  self.weight.element_size() * (self.n_in * self.n_out + M * self.n_in) + out.element_size() * M * self.n_out)
        if fast and few:
            ops.linear_few_rows(x, self.weight, self.bias, out, ctx.stream, epilogue=epi, residual=residual, fold=fold)
        elif fast:
            ops.linear_tensor_cores(x, self.weight, self.bias, out, ctx.status, ctx.stream, epilogue=epi,
                                    residual=residual, fold=fold)
        else:
            ops.linear_generic(x, self.weight, self.bias, out, ctx.stream, epilogue=epi, residual=residual)
        return out
