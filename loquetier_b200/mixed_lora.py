"""The LoRA linear of the Virtualized Module on the B200 SMLM path: the mirror of
``MixedLoraContext``, ``NamedLoraLayer``, ``MixedLoraLinear`` and the weight
preparation of src/loquetier_src/models/mixed_lora.py (:24-64, :78-84, :86-218,
:501-521) - same constructor arguments, same pointer tables, same context fields.

What changes is where the work happens: the per-step segment plan and the adapter
index array are built once per ``MixedLoraContext.update`` and shared by every
LoRA linear of the model; shrink, expand, the per-adapter scale and the add to the
base result run as two kernels that write into the base result in place; the
backward runs native kernels instead of per-partition torch matmuls."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple, Union

import torch
from torch import nn
from torch.autograd.function import Function

from . import ops
from .kernel_utils import BatchLenInfo, _ptr_table, add_lora
from .segments import wants_grouped_plan


class MixedLoraContext:
    """Per-step batch description shared by all LoRA linears (mixed_lora.py:24-64),
    plus the device-side artefacts derived from it once per step."""

    def __init__(self):
        self._blen = None
        self._lora_ids = None
        self._lora_len = None
        self._segment = None
        self._train_idx = []
        self._dev: Dict[Tuple[torch.device, int], dict] = {}

    def update(self, blen: Optional[BatchLenInfo] = None, lora_ids: Optional[List[int]] = None,
               lora_len: Optional[torch.Tensor] = None, segment: Optional[torch.Tensor] = None,
               train_idx: List[int] = []):
        self._blen = blen
        self._lora_ids = lora_ids
        self._lora_len = lora_len
        self._segment = segment
        self._train_idx = train_idx
        self._dev = {}

    blen = property(lambda self: self._blen)
    lora_ids = property(lambda self: self._lora_ids)
    lora_len = property(lambda self: self._lora_len)
    segment = property(lambda self: self._segment)
    train_idx = property(lambda self: self._train_idx)

    def device_state(self, device: torch.device, T: int) -> dict:
        """Segment index pointer, adapter index per segment, train partitions and
        their plans on ``device``; built on first use after ``update``."""
        key = (device, int(T))
        st = self._dev.get(key)
        if st is None:
            seg = self._segment.to(device=device, dtype=torch.int32).contiguous()
            seg_ids = torch.tensor(list(self._lora_ids), dtype=torch.int32, device=device)
            # grouped plan when it helps: decode tokens of one adapter then share its panels wherever they
            # sit in the batch.  The reference keeps `segment` on the device (model_generation.py:279-283):
            # its lengths come back in ONE copy, outside any stream capture (the state is built on the
            # first forward after `update`), never element by element.
            bounds = self._segment.tolist()
            lens = [b - a for a, b in zip(bounds[:-1], bounds[1:])]
            if wants_grouped_plan(lens, list(self._lora_ids)):
                plan = ops.Plan(seg, T, seg_ids=seg_ids, n_table=max(self._lora_ids) + 1)
            else:
                plan = ops.Plan(seg, T)
            st = dict(segment=seg, plan=plan, seg_ids=seg_ids)
            tl = int(self._blen.tlen) if self._blen is not None else 0
            if tl > 0:
                tp = [int(v) for v in self._blen.train_partition]
                part = torch.tensor(tp, dtype=torch.int32, device=device)
                st.update(part=part, part_plan=ops.Plan(part, tl), tlen=tl,
                          part_ids=torch.tensor(list(self._train_idx), dtype=torch.int32, device=device))
            self._dev[key] = st
        return st


@dataclass
class NamedLoraLayer:
    adapter_name: str
    wa: torch.Tensor            # [rank, h_in]
    wb: torch.Tensor            # [h_out, rank]
    dropout: Union[nn.Dropout, nn.Identity]
    scaling: Optional[float] = None


def prepare_weight(weight: torch.Tensor, rank: int, dtype: torch.dtype, device, rank_dim: int = 0,
                   scaling: Optional[float] = None) -> torch.Tensor:
    """Detach, optionally bake the scale in, cast, make contiguous, and zero-pad the
    rank dimension up to the model-wide rank (mixed_lora.py:501-521)."""
    weight = weight.detach()
    if scaling is not None:
        weight = weight * scaling
    if weight.size(rank_dim) == rank:
        return weight.to(dtype=dtype, device=device).contiguous()
    size = list(weight.size())
    size[rank_dim] = rank
    out = torch.zeros(size, dtype=dtype, device=device)
    out[:weight.size(0), :weight.size(1)].copy_(weight)
    return out


class _lora_linear_fn(Function):
    """result += scale * (x . A^T) . B^T over all segments, in place, with the
    native backward over the train partitions."""

    @staticmethod
    def forward(ctx, result, x, mod, st, *trainable):
        v = torch.empty((x.size(0), mod.rank), dtype=x.dtype, device=x.device)
        ops.fwd(result, x, v, mod.wa_ptrs, mod.wb_ptrs, st["plan"], mod.rank, is_row_major=False,
                seg_ids=st["seg_ids"], seg_scale=mod.scaling_f32, accumulate=True)
        ctx.mark_dirty(result)
        ctx.mod, ctx.st, ctx.ntrain = mod, st, len(trainable)
        tl = st.get("tlen", 0)
        ctx.save_for_backward(x[:tl], v[:tl])
        return result

    @staticmethod
    def backward(ctx, grad_out):
        mod, st = ctx.mod, ctx.st
        x, v = ctx.saved_tensors
        tl = st.get("tlen", 0)
        go = grad_out.contiguous()
        grad_x = torch.zeros((go.size(0), x.size(1)), dtype=go.dtype, device=go.device)
        grads: List[Optional[torch.Tensor]] = [None] * ctx.ntrain
        if tl > 0 and ctx.ntrain > 0:
            npart = ctx.ntrain // 2
            dA = [torch.empty_like(mod.adapters[i].wa) for i in mod.root_context.train_idx[:npart]]
            dB = [torch.empty_like(mod.adapters[i].wb) for i in mod.root_context.train_idx[:npart]]
            dv = torch.empty((tl, mod.rank), dtype=go.dtype, device=go.device)
            ops.bwd(grad_x, _ptr_table(dA, go.device), _ptr_table(dB, go.device), dv, go, x.contiguous(),
                    v.contiguous(), mod.wa_ptrs, mod.wb_ptrs, st["part_plan"], mod.rank, is_row_major=False,
                    part_ids=st["part_ids"], part_scale=mod.scaling_f32)
            grads = [g for pair in zip(dA, dB) for g in pair]
        return (grad_out, grad_x, None, None, *grads)


class MixedLoraLinear(nn.Module):
    """Base linear plus the segmented multi-LoRA update (mixed_lora.py:86-218)."""

    def __init__(self, root_context: MixedLoraContext, base_layer: Any, adapters: List[NamedLoraLayer],
                 rank: int, dtype: torch.dtype, is_scaled: bool = False):
        super().__init__()
        self.root_context = root_context
        self.base_layer = base_layer
        self.device = base_layer.weight.device
        self.dtype = dtype
        self.is_scaled = is_scaled
        self.scaling = None
        self.scaling_f32 = None
        self.update_adapters(adapters, rank)

    # -- pointer tables (mixed_lora.py:106-166) ---------------------------------
    def _refresh_tables(self):
        self.wa_ptrs = _ptr_table([a.wa for a in self.adapters], self.device)
        self.wb_ptrs = _ptr_table([a.wb for a in self.adapters], self.device)
        if not self.is_scaled:
            vals = [a.scaling for a in self.adapters]
            self.scaling = torch.tensor(vals, dtype=self.dtype, device=self.device)
            # the kernels take the scale in fp32; it carries the module dtype's rounding
            self.scaling_f32 = self.scaling.to(torch.float32)

    def update_adapters(self, adapters: List[NamedLoraLayer], rank: int):
        self.adapters = adapters
        self.rank = rank
        self._refresh_tables()

    def add_adapter(self, adapter: NamedLoraLayer):
        """The new adapter must have the rank of the existing ones."""
        self.adapters.append(adapter)
        self._refresh_tables()

    def del_adapter(self, adapter_idx: int):
        assert adapter_idx < len(self.adapters)
        del self.adapters[adapter_idx]
        self._refresh_tables()

    def set_trainable(self, train_idx: List[int]):
        for idx in train_idx:
            self.register_parameter(f'lora-{idx}-A', nn.Parameter(self.adapters[idx].wa))
            self.register_parameter(f'lora-{idx}-B', nn.Parameter(self.adapters[idx].wb))

    # -- forward ----------------------------------------------------------------
    def _dropped(self, x, blen, train_idx):
        if blen.tlen <= 0:
            return x
        if all(isinstance(self.adapters[i].dropout, nn.Identity) or not self.adapters[i].dropout.training
               or getattr(self.adapters[i].dropout, "p", 0.0) == 0.0 for i in train_idx):
            return x
        parts = []
        for idx, pi in zip(train_idx, range(len(blen.train_partition) - 1)):
            a, b = blen.train_partition[pi], blen.train_partition[pi + 1]
            parts.append(self.adapters[idx].dropout(x[a:b, :]))
        return torch.cat(parts + [x[blen.tlen:, :]])

    def forward(self, x: torch.Tensor, *args: Any, **kwargs: Any) -> torch.Tensor:
        result = self.base_layer(x, *args, **kwargs)
        out_dtype = result.dtype
        ctxt = self.root_context
        blen, train_idx = ctxt.blen, ctxt.train_idx
        x = self._dropped(x.to(self.dtype), blen, train_idx)
        if not x.is_contiguous():
            x = x.contiguous()
        if result.dtype != self.dtype or not result.is_contiguous():
            result = result.to(self.dtype).contiguous()
        st = ctxt.device_state(x.device, x.size(0))
        trainable = [w for idx in train_idx for w in (self.get_parameter(f'lora-{idx}-A'),
                                                      self.get_parameter(f'lora-{idx}-B'))]
        needs_grad = torch.is_grad_enabled() and (x.requires_grad or result.requires_grad
                                                  or any(w.requires_grad for w in trainable))
        if needs_grad:
            if result.is_leaf and result.requires_grad:
                result = result.clone()
            result = _lora_linear_fn.apply(result, x, self, st, *trainable)
        else:
            v = torch.empty((x.size(0), self.rank), dtype=x.dtype, device=x.device)
            ops.fwd(result, x, v, self.wa_ptrs, self.wb_ptrs, st["plan"], self.rank, is_row_major=False,
                    seg_ids=st["seg_ids"], seg_scale=self.scaling_f32, accumulate=True)
        return result.to(out_dtype)

    def forward_reference_ops(self, x: torch.Tensor, *args: Any, **kwargs: Any) -> torch.Tensor:
        """The reference's own sequence of operator calls (pointer gather, add_lora,
        per-token scale, add; mixed_lora.py:173-218) on the B200 kernels, for
        parity runs that want the reference's rounding points."""
        result = self.base_layer(x, *args, **kwargs)
        out_dtype = result.dtype
        ctxt = self.root_context
        blen, lora_ids, lora_len, train_idx = ctxt.blen, ctxt.lora_ids, ctxt.lora_len, ctxt.train_idx
        segment = ctxt.segment.to(self.device)
        wa_ptr, wb_ptr = self.wa_ptrs[lora_ids], self.wb_ptrs[lora_ids]
        x = self._dropped(x.to(self.dtype), blen, train_idx)
        lora_res = add_lora.apply(
            result.shape, x, wa_ptr, wb_ptr, segment, self.rank, blen.tlen, blen.train_partition,
            *[w for idx in train_idx for w in (self.get_parameter(f'lora-{idx}-A'),
                                              self.get_parameter(f'lora-{idx}-B'))])
        if not self.is_scaled:
            lora_res = lora_res * torch.repeat_interleave(self.scaling[lora_ids], lora_len).unsqueeze(-1)
        return (result + lora_res).to(out_dtype)
