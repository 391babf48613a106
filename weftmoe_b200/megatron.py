"""Megatron-Core routed-MoE adapter over `TensorRuntime`; router, shared experts and DDP stay Megatron's.

Entry points follow the reference's `weftmoe/megatron.py` (`MegatronAdapter(models, max_tokens=, fp8=,
batch_invariant=)` :45-46, `prepare` :94, `pack` :124-136, `weights_updated` :155, `forward_experts`
:164-188, `get_runtime` :190-209, `suspend` :244, `close` :262; autograd function `_Routed` :14-42).
The FP32-master / AReaL weight residency (`bind_fp32_masters`, `weftmoe/_master_weights.py`) is outside this
build's scope.  Megatron-Core is not required to import this module: layers are recognised by their class
name and attributes, which also lets the pure-tensor parts be tested without the framework.
"""
from __future__ import annotations

import os
from types import MethodType

import torch

from .runtime import TensorRuntime

REQUIREMENT = ("WeftMoE requires ETP1, bias-free SwiGLU, separate shared experts, "
               "and no partial MoE checkpoint (full-layer checkpoint is supported)")


def _is_moe_layer(module) -> bool:
    try:
        from megatron.core.transformer.moe.moe_layer import MoELayer
        return isinstance(module, MoELayer)
    except ImportError:
        return type(module).__name__ == "MoELayer"


def _unsupported(layer) -> bool:
    c = layer.config
    get = lambda name, default=None: getattr(c, name, default)
    return bool(get("moe_latent_size") or get("moe_shared_expert_overlap") or get("add_bias_linear")
                or get("expert_tensor_parallel_size", 1) != 1 or getattr(layer, "moe_layer_recompute", False)
                or not get("gated_linear_unit", True) or get("activation_func", torch.nn.functional.silu)
                is not torch.nn.functional.silu or get("moe_apply_probs_on_input")
                or get("activation_func_clamp_value") is not None or get("glu_linear_offset", 0) != 0)


class _ExpertCall:
    """What one routed-expert call has to remember between its forward and its backward."""

    def __init__(self, manager, layer):
        self.manager = manager
        self.runtime = manager.get_runtime(layer)
        self.version_at_forward = manager.weight_version
        self.tape = None

    def gradients(self, dy, parameters):
        manager = self.manager
        if manager.fp8:
            # the FP8 tape references the weights prepared at forward time; an optimizer step in between
            # would make the backward read a different weight version than the forward did
            if manager.weight_version != self.version_at_forward:
                raise RuntimeError("Expert weights changed before FP8 backward")
        else:
            # all layers share one packed buffer pair: put THIS layer's weights back before using it
            manager.pack(parameters)
        return self.runtime.backward_async(self.tape, dy)


class _Routed(torch.autograd.Function):
    """Autograd edge between Megatron's per-expert Parameters and the stacked operator: every Parameter
    is an input of the function, so each receives its own gradient tensor and DDP's hooks fire as usual.
    Inputs: (manager, layer, x, routes, gates, fc1 weights..., fc2 weights...)."""

    @staticmethod
    def forward(ctx, manager, layer, x, routes, gates, *parameters):
        call = _ExpertCall(manager, layer)
        call.tape = manager.forward_experts(layer, x, routes, gates, parameters)
        ctx.call = call
        # saving the Parameters lets autograd itself flag an in-place update made before backward
        ctx.save_for_backward(*parameters)
        return call.tape.output

    @staticmethod
    def backward(ctx, dy):
        call, ctx.call = ctx.call, None
        dx, dgates, dw1, dw2 = call.gradients(dy, ctx.saved_tensors)
        per_expert = [*dw1.unbind(0), *dw2.unbind(0)]
        # one entry per forward input: manager, layer, x, routes, gates, then the Parameters
        return (None, None, dx, None, dgates, *per_expert)


class MegatronAdapter:
    def __init__(self, models, *, max_tokens, fp8=None, batch_invariant=True):
        self.max_tokens = max_tokens
        self.batch_invariant = batch_invariant
        self.fp8 = os.environ.get("WEFTMOE_FP8", "0") == "1" if fp8 is None else fp8
        self.fp8_weights = {}
        self.weight_version = 0
        self.runtime = None
        self.session = None
        self.packed = {}
        self.layers = []
        self._optimizer_hook = None
        self._models = tuple(models)
        for model in self._models:
            if getattr(getattr(model, "ddp_config", None), "overlap_param_gather", False):
                raise ValueError("WeftMoE requires overlap_param_gather=False")
            for layer in model.modules():
                if not _is_moe_layer(layer):
                    continue
                if _unsupported(layer):
                    raise ValueError(REQUIREMENT)
                self.layers.append(layer)
                layer.forward = MethodType(self._make_forward(), layer)
        if not self.layers:
            raise ValueError("No Megatron MoE layers found")

    # ------------------------------------------------------------------ weights
    @staticmethod
    def _parameters(layer):
        """[fc1 weight of expert 0..E_local-1, fc2 weight of expert 0..E_local-1]."""
        return [getattr(linear, f"weight{i}")
                for linear in (layer.experts.linear_fc1, layer.experts.linear_fc2)
                for i in range(layer.num_local_experts)]

    def pack(self, parameters):
        """The operator wants [E,2I,H] and [E,H,I]; Megatron keeps one [2I,H] and one [H,I] Parameter per
        local expert.  Copies them, expert by expert, into a buffer pair that is allocated once per
        (expert count, shapes) and shared by all layers.  Returns (w1, w2)."""
        half = len(parameters) // 2
        fc1, fc2 = parameters[:half], parameters[half:]
        key = (half, tuple(fc1[0].shape), tuple(fc2[0].shape))
        buffers = self.packed.get(key)
        if buffers is None:
            buffers = tuple(group[0].new_empty((half, *group[0].shape)) for group in (fc1, fc2))
            self.packed[key] = buffers
        with torch.no_grad():  # plain buffers: the autograd edge to the Parameters is _Routed
            for buffer, group in zip(buffers, (fc1, fc2)):
                torch._foreach_copy_(list(buffer.unbind(0)), list(group))   # one multi-tensor copy
        return buffers

    def bind_optimizer(self, optimizer):
        """Reuse prepared FP8 weights until this torch.optim.AdamW steps."""
        register = getattr(optimizer, "register_step_post_hook", None)
        if not isinstance(optimizer, torch.optim.AdamW) or not callable(register):
            raise TypeError("bind_optimizer requires torch.optim.AdamW with register_step_post_hook")
        if self._optimizer_hook is not None:
            self._optimizer_hook.remove()
        self._optimizer_hook = register(lambda *_: self.weights_updated())
        self.weights_updated()

    def bind_fp32_masters(self, optimizer):
        raise NotImplementedError("FP32-master FP8 residency (AReaL) is outside this build's scope")

    def weights_updated(self):
        """Invalidate after optimizer/checkpoint writes, including .data copies."""
        self.weight_version += 1
        self.fp8_weights.clear()

    # ------------------------------------------------------------------ compute
    def prepare(self):
        """Validate and allocate the communication context before rollout starts."""
        self.get_runtime(self.layers[0])

    def get_runtime(self, layer):
        if self.runtime is None:
            cfg = layer.config
            self.runtime = TensorRuntime(
                group=layer.ep_group, experts=cfg.num_moe_experts, top_k=cfg.moe_router_topk,
                hidden=cfg.hidden_size, intermediate=cfg.moe_ffn_hidden_size, max_tokens=self.max_tokens,
                max_rows=self.max_tokens * cfg.moe_router_topk * 2 + layer.num_local_experts * 128,
                training=True, max_saved=len(self.layers) + 8, session=self.session,
                fp8_workspace=self.fp8, batch_invariant=self.batch_invariant)
            self.session = self.runtime.native.session()
        return self.runtime

    def forward_experts(self, layer, x, routes, gates, parameters, *, retain=True):
        runtime = self.get_runtime(layer)
        if not self.fp8:
            return runtime.forward_async(x, routes, gates, *self.pack(parameters), retain_backward_state=retain)
        from .fp8 import prepare_fp8_weights
        versions = tuple(p._version for p in parameters)
        cacheable = self._optimizer_hook is not None
        entry = self.fp8_weights.get(layer) if cacheable else None
        if entry is None or entry[0] != versions:
            entry = (versions, prepare_fp8_weights(*self.pack(parameters), training=True,
                                                   version=self.weight_version))
            if cacheable:
                self.fp8_weights[layer] = entry
        return runtime.forward_fp8(x, routes, gates, entry[1], synchronize=False,
                                   retain_backward_state=retain, weight_grad_dtype=torch.bfloat16)

    def _make_forward(self):
        manager = self

        def forward(layer, hidden_states, intermediate_tensors=None, padding_mask=None):
            if intermediate_tensors is not None:
                raise ValueError("WeftMoE replaces the whole routed path; partial MoE execution is unsupported")
            if padding_mask is not None:
                padding_mask = padding_mask.transpose(0, 1).bool()
            shared = layer.shared_experts_compute(hidden_states)
            probabilities, _ = layer.route(hidden_states, padding_mask)
            gates, routes = probabilities.topk(layer.config.moe_router_topk, dim=-1)
            inputs = (hidden_states.reshape(-1, hidden_states.shape[-1]).contiguous(),
                      routes.int().contiguous(), gates.float().contiguous())
            parameters = manager._parameters(layer)
            if torch.is_grad_enabled():  # Megatron's full-layer checkpoint runs its first pass under no_grad
                output = _Routed.apply(manager, layer, *inputs, *parameters)
            else:
                output = manager.forward_experts(layer, *inputs, parameters, retain=False).output
            output = output.view_as(hidden_states)
            return (output if shared is None else output + shared), None

        return forward

    # ------------------------------------------------------------------ lifecycle
    def suspend(self):
        """Release idle training workspaces while rollout owns the GPUs."""
        if self.runtime is not None:
            torch.cuda.synchronize()
            self.runtime.drain()
            if self.runtime.native.usage()["notify_slots_in_use"]:
                raise RuntimeError("Cannot offload WeftMoE while autograd still owns saved X/AB")
            self.runtime.close()
            self.runtime = None
        self.weights_updated()
        self.packed.clear()

    def close(self):
        """Release buffers and the session when the training engine is destroyed."""
        self.suspend()
        self.fp8_weights.clear()
        self.session = None
        if self._optimizer_hook is not None:
            self._optimizer_hook.remove()
            self._optimizer_hook = None
        if torch.cuda.is_available():
            torch.cuda.empty_cache()
