"""Which path a linear-attention layer's step takes, decided from the engine's attention metadata alone.

The decision is separated from its execution so that it can be stated, and tested, without a serving engine: the
adapters in gdn.py and glm.py ask `plan_step(...)` and then carry the plan out with the engine's own tensors.  The
conditions are the reference plugin's (leapquant/vllm/gdn.py:53-78 for Gated DeltaNet layers, leapquant/vllm/glm.py:25-75
for Kimi Delta Attention layers):

  ENGINE       no metadata for this layer (profiling / warm-up runs), or nothing to do: the engine's own forward runs.
  DECODE       only decode tokens: conv1d update, then one decode call on the 8-bit state.
  MIXED        prefill and decode tokens in one step: the decode tokens go through the 8-bit state, the prefill slots take
               an fp32 round trip (dequantize -> the engine's prefill kernel -> quantize).
  ROUND_TRIP   speculative decoding (or an engine whose metadata does not separate the prefill slots): every slot the step
               touches takes the fp32 round trip around the engine's own forward.
"""
import enum
from dataclasses import dataclass

import torch


class Route(enum.Enum):
    ENGINE = "engine"
    DECODE = "decode"
    MIXED = "mixed"
    ROUND_TRIP = "round_trip"


@dataclass
class StepPlan:
    route: Route
    slots: "torch.Tensor | None" = None       # slots that take the fp32 round trip (MIXED: prefill slots; ROUND_TRIP: all touched)


def touched_slots(md):
    """Every state slot the step reads or writes (speculative and non-speculative sequences), clamped at the null slot."""
    parts = [t.reshape(-1) for t in (getattr(md, "non_spec_state_indices_tensor", None),
                                     getattr(md, "spec_state_indices_tensor", None)) if t is not None]
    if not parts:
        return None
    return torch.cat(parts).clamp(min=0)


def plan_gdn_step(md, packed_decode=True):
    """Gated DeltaNet layer (reference leapquant/vllm/gdn.py:53-78).  `md` is the layer's GDNAttentionMetadata or None."""
    if md is None:
        return StepPlan(Route.ENGINE)
    spec = md.spec_sequence_masks is not None
    if packed_decode and not spec and md.num_prefills == 0 and md.num_decodes > 0:
        return StepPlan(Route.DECODE)
    prefill_slots = getattr(md, "prefill_state_indices", None)
    if not spec and prefill_slots is not None:
        return StepPlan(Route.MIXED, prefill_slots.reshape(-1).clamp(min=0))
    slots = touched_slots(md)
    if slots is None:
        return StepPlan(Route.ENGINE)
    return StepPlan(Route.ROUND_TRIP, slots)


def plan_kda_step(md):
    """Kimi Delta Attention layer (reference leapquant/vllm/glm.py:25-75)."""
    if md is None or md.num_actual_tokens == 0:
        return StepPlan(Route.ENGINE)
    if md.spec_sequence_masks is not None and md.num_spec_decodes > 0:
        return StepPlan(Route.ROUND_TRIP, touched_slots(md))
    if md.num_prefills > 0:
        return StepPlan(Route.MIXED, md.prefill_state_indices.clamp(min=0))
    return StepPlan(Route.DECODE)


def layer_metadata(forward_context, prefix):
    """The metadata object of the layer named `prefix`, or None when the engine runs without one (profiling, warm-up)."""
    raw = forward_context.attn_metadata
    return raw.get(prefix) if isinstance(raw, dict) else None


def conv_weight_2d(conv):
    """A depthwise conv1d module's weight [dim, 1, width] as the [dim, width] matrix the conv-update kernels take."""
    w = conv.weight
    return w.view(w.size(0), w.size(2))
