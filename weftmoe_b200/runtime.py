"""Tensor API of the routed-MoE expert operator: one persistent native workspace per EP group.

Mirror of the reference's `weftmoe/runtime.py` (`TensorRuntime` :23-464, `_MoE` :467-479, `moe`
:506-512) with the same constructor keywords, method names, argument meaning and error
behaviour, over the C ABI in include/weftmoe_b200.h.  `NativeRuntime` plays the part of the
reference's Blackwell backend object (`weftmoe/blackwell.py:51-178`).  PyTorch is used for
tensors, streams and the bootstrap collectives only; all compute is in libweftmoe_b200.so.

Preparation is collective: all ranks of the group construct the runtime and call layers in the
same order.  Expert weights are BF16 [local_experts, 2*intermediate, hidden] (rows 0..I-1 gate,
I..2I-1 up) and [local_experts, hidden, intermediate].
"""
from __future__ import annotations

import ctypes
import socket
import weakref
from dataclasses import dataclass

import torch
import torch.distributed as dist

from . import _lib


# Routes (tokens * top_k) per rank that the single-launch planner of libweftmoe_b200 handles
# (kSmallPlanRoutes in csrc/route.h); a decode_only runtime never exceeds it.
DECODE_MAX_ROUTES = 4096


class SingleRankGroup:
    """Stand-in for a one-rank process group, so EP1 needs no torch.distributed initialisation.

    The reference forms its EP1 groups with `dist.new_subgroups(group_size=1)`
    (tests/torchrun_sm100_invariant.py:27); a real one-rank ProcessGroup works here too."""

    def size(self):
        return 1

    def rank(self):
        return 0


class _Collectives:
    """The few bootstrap collectives the runtime needs, over a real group or SingleRankGroup."""

    def __init__(self, group):
        self.group = group
        self.single = isinstance(group, SingleRankGroup)
        self.rank = 0 if self.single else dist.get_rank(group)
        self.world = 1 if self.single else dist.get_world_size(group)

    def all_gather_object(self, value):
        if self.single:
            return [value]
        out = [None] * self.world
        dist.all_gather_object(out, value, group=self.group)
        return out

    def barrier(self):
        if not self.single:
            dist.barrier(group=self.group)


def agree_on_preparation(collectives, error):
    """Every rank reports the outcome of its local preparation (None or a message); if any rank
    failed, ALL ranks raise, so no rank is left waiting in the handle exchange that follows
    (reference: weftmoe/runtime.py:181-188).  ValueError only if every failure was a ValueError."""
    errors = collectives.all_gather_object(error)
    if any(errors):
        kind = ValueError if all(e is None or e.startswith("ValueError") for e in errors) else RuntimeError
        raise kind(f"collective preparation failed: {[e for e in errors if e]}")


def exchange_handles(collectives, mine: bytes) -> bytes:
    """All-gather the ranks' CUDA-IPC handles; returns them concatenated in rank order."""
    handles = collectives.all_gather_object(bytes(mine))
    if any(len(h) != len(mine) for h in handles):
        raise RuntimeError("EP ranks exported IPC handles of different sizes")
    return b"".join(handles)


@dataclass(eq=False)
class Tape:
    """Result of a training forward: `output` plus the cache backward consumes
    (reference: weftmoe/blackwell_backward.py:14-17; src/python/runtime.cpp:880-906)."""
    output: torch.Tensor
    state: tuple | None = None

    @property
    def tensor_bytes(self):
        return 0 if self.state is None else self.state[0].numel()

    @property
    def saved_x_bytes(self):
        return 0 if self.state is None else self.state[-1]


class NativeRuntime:
    """Owner of one `wm_runtime` handle; serialised on the supplied CUDA stream."""

    PRECISIONS = {"bf16": 0, "fp8": 1, "nvfp4": 2}

    def __init__(self, collectives, experts, top_k, hidden, intermediate, max_tokens, max_rows,
                 stream, training, max_saved, precision="bf16"):
        self.lib = _lib.load()
        self.col = collectives
        # A legacy default stream cannot join a caller's CUDA Graph capture
        # (same rule as weftmoe/blackwell.py:60-64).
        self.stream = (torch.cuda.Stream(device=stream.device)
                       if not training and stream == torch.cuda.default_stream(stream.device)
                       else stream)
        self.training, self.max_saved = training, max_saved
        self.tapes = weakref.WeakSet()
        self.plans = {}          # (layer, tokens) -> addresses a replayable inference was prepared with
        self.shape = (experts, top_k, hidden, intermediate)
        self.local_experts = experts // collectives.world
        config = _lib.WmConfig(rank=collectives.rank, world=collectives.world, experts=experts,
                               top_k=top_k, hidden=hidden, intermediate=intermediate,
                               max_tokens=max_tokens, max_rows=max_rows, training=int(training),
                               reserved=self.PRECISIONS[precision])
        self.precision = precision
        self.scales = None  # NVFP4Scales, set by TensorRuntime for precision "nvfp4"
        handle = ctypes.c_void_p()
        # Agree on the outcome of local preparation before any rank touches a peer mapping.
        error = None
        try:
            with torch.cuda.device(stream.device):
                _lib.check(self.lib.wm_runtime_create(ctypes.byref(config), ctypes.byref(handle)))
        except (ValueError, RuntimeError) as exc:
            error = f"{type(exc).__name__}: {exc}"
        try:
            agree_on_preparation(collectives, error)
        except Exception:
            if handle:
                self.lib.wm_runtime_destroy(handle)
            raise
        self.handle = handle
        self.sizes = _lib.WmSizes()
        _lib.check(self.lib.wm_runtime_sizes(self.handle, ctypes.byref(self.sizes)))
        if collectives.world > 1:
            n = self.sizes.ipc_handle_bytes
            mine = ctypes.create_string_buffer(n)
            _lib.check(self.lib.wm_runtime_export_handle(self.handle, mine, n))
            blob = exchange_handles(collectives, mine.raw)
            with torch.cuda.device(stream.device):
                _lib.check(self.lib.wm_runtime_import_peers(self.handle, blob, len(blob)))
            collectives.barrier()

    # ------------------------------------------------------------------ helpers
    def _require(self):
        if self.handle is None:
            raise RuntimeError("WeftMoE runtime is closed")

    def _poll(self):
        code = ctypes.c_int32(0)
        _lib.check(self.lib.wm_status_poll(self.handle, ctypes.byref(code), self.stream.cuda_stream))
        _lib.check(code.value)

    def _run(self, x, routes, gates, w1, w2, *, save=False):
        self._require()
        caller = torch.cuda.current_stream()
        if caller.device != self.stream.device or x.device != self.stream.device:
            raise ValueError("Workspace and tensors must share the current device")
        if caller != self.stream:
            self.stream.wait_stream(caller)
        with torch.cuda.stream(self.stream):
            y = torch.empty_like(x)
            blob = None
            if save:
                if len(self.tapes) >= self.max_saved:
                    raise RuntimeError("Blackwell training tape capacity exhausted")
                blob = torch.empty(self.sizes.tape_bytes, dtype=torch.uint8, device=x.device)
            _lib.check(self.lib.wm_forward(self.handle, _lib.ptr(x), _lib.ptr(routes), _lib.ptr(gates),
                                           _lib.ptr(w1), _lib.ptr(w2), x.shape[0], _lib.ptr(y),
                                           _lib.ptr(blob), self.stream.cuda_stream))
            if caller != self.stream:
                for tensor in (x, routes, gates, w1, w2):
                    tensor.record_stream(self.stream)
                y.record_stream(caller)
        if caller != self.stream:
            caller.wait_stream(self.stream)
        if not save:
            return y
        saved_x = 2 * self.sizes.row_capacity * self.shape[2]
        tape = Tape(y, (blob, w1, w2, x.shape[0], saved_x))
        self.tapes.add(tape)
        return tape

    # ------------------------------------------------------------------ quantised inference
    def _run_quantized(self, x, routes, gates, packed, save=False):
        """packed: (w1 data, w1 scale chunks, w2 data, w2 scale chunks, x_scale, w1_scale, u_scale, w2_scale).
        x: BF16 [T, H], or (FP8 only) an FP8Tensor of that shape quantised 1 x 128, whose bytes and scales
        are used as they are."""
        self._require()
        from .fp8 import FP8Tensor
        source = x if isinstance(x, FP8Tensor) else None
        if source is not None:
            x = source.data
        caller = torch.cuda.current_stream()
        if caller.device != self.stream.device or x.device != self.stream.device:
            raise ValueError("Workspace and tensors must share the current device")
        if caller != self.stream:
            self.stream.wait_stream(caller)
        with torch.cuda.stream(self.stream):
            y = torch.empty(tuple(x.shape), dtype=torch.bfloat16, device=x.device)
            blob = None
            if save:
                if len(self.tapes) >= self.max_saved:
                    raise RuntimeError("Blackwell training tape capacity exhausted")
                blob = torch.empty(self.sizes.tape_bytes, dtype=torch.uint8, device=x.device)
            w1, w1_sf, w2, w2_sf, sx, s1, su, s2 = packed[:8]
            weights = _lib.WmQuantWeights(w1=w1.data_ptr(), w1_sf=w1_sf.data_ptr(), w2=w2.data_ptr(),
                                          w2_sf=w2_sf.data_ptr(), x_scale=sx, w1_scale=s1, u_scale=su, w2_scale=s2)
            if len(packed) > 8:   # FP8 block scales with mantissas: the FP32 scales go along
                weights.w1_scales, weights.w2_scales = packed[8].data_ptr(), packed[9].data_ptr()
            if source is not None:
                weights.source_q, weights.source_scales = source.data.data_ptr(), source.scales.data_ptr()
            _lib.check(self.lib.wm_forward_quantized(self.handle, None if source is not None else _lib.ptr(x),
                                                     _lib.ptr(routes), _lib.ptr(gates),
                                                     ctypes.byref(weights), x.shape[0], _lib.ptr(y),
                                                     _lib.ptr(blob), self.stream.cuda_stream))
            if caller != self.stream:
                held = (x, routes, gates, w1, w1_sf, w2, w2_sf) + ((source.scales,) if source is not None else ())
                for tensor in held:
                    tensor.record_stream(self.stream)
                y.record_stream(caller)
        if caller != self.stream:
            caller.wait_stream(self.stream)
        return (y, blob) if save else y

    def _fp8_packed(self, weights):
        """UE8M0 scale-factor chunks of prepared FP8 weights (packed once per weight version)."""
        cached = getattr(weights, "_wm_chunks", None)
        if cached is None:
            chunks = []
            for w in (weights.w1, weights.w2):
                e, n, k = w.shape
                out = torch.empty(e * n // 128, k // 128, 128, dtype=torch.int32, device=w.data.device)
                _lib.check(self.lib.wm_fp8_pack_weight_scales(_lib.ptr(w.scales), e * n, k // 128, _lib.ptr(out),
                                                              torch.cuda.current_stream().cuda_stream))
                chunks.append(out)
            cached = tuple(chunks)
            object.__setattr__(weights, "_wm_chunks", cached)
        packed = (weights.w1.data, cached[0], weights.w2.data, cached[1], 1.0, 1.0, 1.0, 1.0)
        if getattr(weights, "scale_mantissas", False):
            packed += (weights.w1.scales, weights.w2.scales)
        return packed

    def _fp8_packed_transposed(self, weights):
        """The same for W1^T / W2^T (backward operands)."""
        cached = getattr(weights, "_wm_chunks_t", None)
        if cached is None:
            chunks = []
            for w in (weights.w1_t, weights.w2_t):
                e, n, k = w.shape
                out = torch.empty(e * n // 128, k // 128, 128, dtype=torch.int32, device=w.data.device)
                _lib.check(self.lib.wm_fp8_pack_weight_scales(_lib.ptr(w.scales), e * n, k // 128, _lib.ptr(out),
                                                              torch.cuda.current_stream().cuda_stream))
                chunks.append(out)
            cached = tuple(chunks)
            object.__setattr__(weights, "_wm_chunks_t", cached)
        return weights.w1_t.data, cached[0], weights.w2_t.data, cached[1]

    def forward_fp8(self, x, routes, gates, weights, synchronize, retain_backward_state, fp32_wgrad):
        if retain_backward_state and self.training:
            y, blob = self._run_quantized(x, routes, gates, self._fp8_packed(weights), save=True)
            tape = Tape(y, (blob, weights, fp32_wgrad, x.shape[0], self.sizes.row_capacity * self.shape[2]))
            self.tapes.add(tape)
        else:
            tape = Tape(self._run_quantized(x, routes, gates, self._fp8_packed(weights)))
        if synchronize:
            self._poll()
        return tape

    def _backward_fp8(self, tape, dy):
        from .fp8 import FP8Tensor
        blob, weights, fp32_wgrad, tokens, _ = tape.state
        source = dy if isinstance(dy, FP8Tensor) else None
        if source is not None:
            if tuple(source.shape) != tuple(tape.output.shape) or source.data.device != blob.device:
                raise ValueError("Backward requires dY matching the forward output")
            dy = source.data
        elif dy.dtype != torch.bfloat16 or dy.shape != tape.output.shape or dy.device != blob.device:
            raise ValueError("Backward requires BF16 dY matching the forward output")
        weights._validate_version(training=True)
        w1t, w1t_sf, w2t, w2t_sf = self._fp8_packed_transposed(weights)
        e, k = self.local_experts, self.shape[1]
        _, _, hidden, inter = self.shape
        dx = torch.empty(tuple(dy.shape), dtype=torch.bfloat16, device=dy.device)
        dgates = torch.empty((tokens, k), dtype=torch.float32, device=dy.device)
        wgrad = torch.float32 if fp32_wgrad else torch.bfloat16   # FP32: the accumulators, unrounded
        dw1 = torch.empty((e, 2 * inter, hidden), dtype=wgrad, device=dy.device)
        dw2 = torch.empty((e, hidden, inter), dtype=wgrad, device=dy.device)
        packed = _lib.WmQuantWeights(w1=w1t.data_ptr(), w1_sf=w1t_sf.data_ptr(), w2=w2t.data_ptr(),
                                     w2_sf=w2t_sf.data_ptr(), x_scale=1.0, w1_scale=1.0, u_scale=1.0, w2_scale=1.0,
                                     wgrad_f32=int(bool(fp32_wgrad)))
        if source is not None:
            packed.source_q, packed.source_scales = source.data.data_ptr(), source.scales.data_ptr()
        if getattr(weights, "scale_mantissas", False):
            packed.w1_scales, packed.w2_scales = weights.w1_t.scales.data_ptr(), weights.w2_t.scales.data_ptr()
        _lib.check(self.lib.wm_backward_quantized(self.handle, _lib.ptr(blob),
                                                  None if source is not None else _lib.ptr(dy), ctypes.byref(packed),
                                                  tokens, _lib.ptr(dx), _lib.ptr(dgates), _lib.ptr(dw1),
                                                  _lib.ptr(dw2), self.stream.cuda_stream))
        tape.state = None
        self.tapes.discard(tape)
        return dx, dgates, dw1, dw2

    def inference(self, x, routes, gates, weights, x_scale, intermediate_scale):
        """NVFP4 inference with prepared weights (reference: NVFP4Runtime.inference, weftmoe/nvfp4.py:252-278)."""
        (w1, w1_sf), (w2, w2_sf) = weights.fc1, weights.fc2
        return self._run_quantized(x, routes, gates, (w1, w1_sf, w2, w2_sf, x_scale, weights.tensor_scales[0],
                                                      intermediate_scale, weights.tensor_scales[1]))

    # ------------------------------------------------------------------ training
    def forward_async(self, x, routes, gates, w1, w2, retain_backward_state=True):
        if self.precision == "nvfp4":
            return self._forward_nvfp4(x, routes, gates, w1, w2, retain_backward_state)
        if self.training and retain_backward_state:
            return self._run(x, routes, gates, w1, w2, save=True)
        return Tape(self._run(x, routes, gates, w1, w2))

    # NVFP4 training (reference: NVFP4Runtime.forward / weftmoe/nvfp4_backward.py): BF16 master weights are
    # quantised block-16 along the reduction axis of each contraction, forward layout in the forward
    # pass and transposed in the backward pass, with the runtime's layer scales.
    def _nvfp4_weight_version(self, w1, w2):
        """Identity of one version of the BF16 master weights, or None when it cannot be tracked (inference
        tensors carry no in-place version counter).  The quantised forward and transposed layouts are kept
        per version, so the masters are quantised once per optimizer step, not once per call."""
        if w1.is_inference() or w2.is_inference():
            return None
        return (w1.data_ptr(), w1._version, w2.data_ptr(), w2._version, tuple(self.scales))

    def _forward_nvfp4(self, x, routes, gates, w1, w2, retain):
        from .nvfp4 import prepare_nvfp4_weights
        s = self.scales
        version = self._nvfp4_weight_version(w1, w2)
        cache = getattr(self, "_nvfp4_cache", None)
        if version is None or cache is None or cache["version"] != version:
            cache = dict(version=version, forward=prepare_nvfp4_weights(w1, w2, weight_scales=(s.w1, s.w2)),
                         transposed=None)
            self._nvfp4_cache = cache
        q = cache["forward"]
        packed = (q.fc1[0], q.fc1[1], q.fc2[0], q.fc2[1], s.x, s.w1, s.intermediate, s.w2)
        if self.training and retain:
            y, blob = self._run_quantized(x, routes, gates, packed, save=True)
            tape = Tape(y, (blob, w1, w2, x.shape[0], self.sizes.row_capacity * self.shape[2] // 2))
            self.tapes.add(tape)
            return tape
        return Tape(self._run_quantized(x, routes, gates, packed))

    def _backward_nvfp4(self, tape, dy):
        from .nvfp4 import quantize_nvfp4
        blob, w1, w2, tokens, _ = tape.state
        if dy.dtype != torch.bfloat16 or dy.shape != tape.output.shape or dy.device != blob.device:
            raise ValueError("Backward requires BF16 dY matching the forward output")
        s = self.scales
        e, k = self.local_experts, self.shape[1]
        _, _, hidden, inter = self.shape
        version = self._nvfp4_weight_version(w1, w2)
        cache = getattr(self, "_nvfp4_cache", None)
        if version is not None and cache is not None and cache["version"] == version and cache["transposed"]:
            w1t_q, w1t_sf, w2t_q, w2t_sf = cache["transposed"]
        else:
            w1t = w1.transpose(1, 2).contiguous().view(e * hidden, 2 * inter)     # [E*H, 2I]: reduce over 2I
            w2t = w2.transpose(1, 2).contiguous().view(e * inter, hidden)         # [E*I, H]:  reduce over H
            w1t_q, w1t_sf = quantize_nvfp4(w1t, s.w1, chunked=True)
            w2t_q, w2t_sf = quantize_nvfp4(w2t, s.w2, chunked=True)
            if version is not None and cache is not None and cache["version"] == version:
                cache["transposed"] = (w1t_q, w1t_sf, w2t_q, w2t_sf)
        dx = torch.empty_like(dy)
        dgates = torch.empty((tokens, k), dtype=torch.float32, device=dy.device)
        dw1, dw2 = torch.empty_like(w1), torch.empty_like(w2)
        packed = _lib.WmQuantWeights(w1=w1t_q.data_ptr(), w1_sf=w1t_sf.data_ptr(), w2=w2t_q.data_ptr(),
                                     w2_sf=w2t_sf.data_ptr(), x_scale=s.x, w1_scale=s.w1, u_scale=s.intermediate,
                                     w2_scale=s.w2, dy_scale=s.dy, dab_scale=s.dgate_up)
        _lib.check(self.lib.wm_backward_quantized(self.handle, _lib.ptr(blob), _lib.ptr(dy), ctypes.byref(packed),
                                                  tokens, _lib.ptr(dx), _lib.ptr(dgates), _lib.ptr(dw1),
                                                  _lib.ptr(dw2), self.stream.cuda_stream))
        for t in (w1t_q, w1t_sf, w2t_q, w2t_sf):
            t.record_stream(self.stream)
        tape.state = None
        self.tapes.discard(tape)
        return dx, dgates, dw1, dw2

    def forward(self, x, routes, gates, w1, w2):
        tape = self.forward_async(x, routes, gates, w1, w2)
        self._poll()
        return tape

    def backward_async(self, tape, dy):
        self._require()
        if tape not in self.tapes or tape.state is None:
            raise RuntimeError("Backward requires a live training tape from this runtime")
        if self.precision == "fp8":
            return self._backward_fp8(tape, dy)
        if self.precision == "nvfp4":
            return self._backward_nvfp4(tape, dy)
        blob, w1, w2, tokens, _ = tape.state
        if dy.dtype != torch.bfloat16 or dy.shape != tape.output.shape or dy.device != blob.device:
            raise ValueError("Backward requires BF16 dY matching the forward output")
        k = self.shape[1]
        dx = torch.empty_like(dy)
        dgates = torch.empty((tokens, k), dtype=torch.float32, device=dy.device)
        dw1, dw2 = torch.empty_like(w1), torch.empty_like(w2)
        _lib.check(self.lib.wm_backward(self.handle, _lib.ptr(blob), _lib.ptr(dy), _lib.ptr(w1),
                                        _lib.ptr(w2), tokens, _lib.ptr(dx), _lib.ptr(dgates),
                                        _lib.ptr(dw1), _lib.ptr(dw2), self.stream.cuda_stream))
        tape.state = None
        self.tapes.discard(tape)
        return dx, dgates, dw1, dw2

    def backward(self, tape, dy):
        result = self.backward_async(tape, dy)
        self._poll()
        return result

    # ------------------------------------------------------------------ inference
    def graph_forward(self, layer, x, routes, gates, w1, w2, caller_stream, fp8_weights=None):
        """Replayable inference of one (layer, token count) "plan" (reference: Runtime::graph_forward,
        src/python/runtime.cpp:554-616).  The forward itself enqueues only stream-ordered kernels, so a
        caller's capture records it directly; what a plan keeps is the reference's contract around it:
        the first call of a (layer, tokens) pair must come outside capture (warm-up), and later calls must
        present the same input, route, gate and weight addresses, because a captured graph replays the
        addresses it was captured with.  invalidate_inference_layer(layer) forgets the layer's plans."""
        if self.training:
            raise ValueError("graph_forward is inference-only")
        from .fp8 import FP8Tensor
        prequantised = isinstance(x, FP8Tensor)
        source = x.data if prequantised else x             # BF16 tensor, or the bytes of an FP8Tensor
        scales = x.scales.data_ptr() if prequantised else 0
        key = (layer, source.shape[0])
        record = (source.data_ptr(), scales, routes.data_ptr(), gates.data_ptr(), w1.data_ptr(), w2.data_ptr(),
                  None if fp8_weights is None else id(fp8_weights))
        plan = self.plans.get(key)
        if plan is None:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("Warm every inference layer/token bucket before outer graph capture")
            plan = self.plans[key] = record
        if plan[:4] != record[:4]:
            raise RuntimeError("Inference input addresses changed: use stable CUDA Graph buffers or call "
                               "invalidate_inference_layer(layer) before re-preparation")
        if plan[6] != record[6]:
            raise RuntimeError("Weight format/version changed: invalidate inference layer before re-preparation")
        if plan[4:6] != record[4:6]:
            raise RuntimeError("Expert addresses changed: discard outer graphs and call "
                               "invalidate_inference_layer(layer) before re-preparation")
        if fp8_weights is not None:
            return self._run_quantized(x, routes, gates, self._fp8_packed(fp8_weights))
        return self._run(x, routes, gates, w1, w2)

    def eager_inference_async(self, x, routes, gates, w1, w2, caller_stream, layer=None):
        return self._run(x, routes, gates, w1, w2)

    def eager_inference(self, x, routes, gates, w1, w2, caller_stream, layer=None):
        output = self._run(x, routes, gates, w1, w2)
        self._poll()
        return output

    def invalidate_inference_layer(self, layer, caller_stream):
        """Forget the plans of `layer` (its buffers or weights are about to change); graphs captured with
        them must be discarded by the caller.  Waits for the layer's work in flight first."""
        self.stream.synchronize()
        for key in [k for k in self.plans if k[0] == layer]:
            del self.plans[key]

    # ------------------------------------------------------------------ lifecycle
    def drain_eager_inference(self):
        if self.handle is not None:
            self._poll()

    def drain_training(self):
        if self.handle is not None:
            self._poll()

    def usage(self):
        return dict(notify_slots_in_use=len(self.tapes), symmetric_bytes=int(self.sizes.arena_bytes),
                    scratch_bytes=int(self.sizes.scratch_bytes), tape_bytes=int(self.sizes.tape_bytes),
                    row_capacity=int(self.sizes.row_capacity))

    def session(self):
        return None

    # ------------------------------------------------------------------ instrumentation
    def enable_timing(self, enable=True):
        """Bracket every stage of forward/backward with CUDA events on the runtime's stream."""
        self._require()
        _lib.check(self.lib.wm_runtime_enable_timing(self.handle, int(enable)))

    def read_timing(self, reset=True):
        """{stage name: (summed milliseconds, calls)} of the calls made since the last reset."""
        self._require()
        n = self.lib.wm_stage_count()
        ms = (ctypes.c_double * n)()
        calls = (ctypes.c_longlong * n)()
        _lib.check(self.lib.wm_runtime_read_timing(self.handle, ms, calls, int(reset)))
        return {self.lib.wm_stage_name(k).decode(): (ms[k], calls[k]) for k in range(n)}

    def launch_count(self):
        return int(self.lib.wm_launch_count())

    def retire_peer_mappings(self):
        if self.handle is not None:
            self.lib.wm_runtime_retire_peers(self.handle)

    def destroy(self):
        if self.handle is not None:
            self.lib.wm_runtime_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass


class TensorRuntime:
    def __init__(
        self,
        *,
        group,
        experts: int,
        top_k: int,
        hidden: int,
        intermediate: int,
        max_tokens: int,
        max_rows: int,
        training: bool,
        max_saved: int = 64,
        stream=None,
        input_layout: str = "dp",
        interconnect: str | None = None,
        decode_only: bool = False,
        fp8_workspace: bool = False,
        precision: str | None = None,
        nvfp4_scales=None,
        session=None,
        batch_invariant: bool = True,
        allow_unvalidated_shape: bool = False,
        _native_factory=None,
    ):
        if group is None:
            raise ValueError("Pass the explicit expert process group")
        self.group = group
        col = self._collectives = _Collectives(group)
        self.rank, self.world = col.rank, col.world
        hosts = col.all_gather_object(socket.gethostname())
        ordered_hosts = list(dict.fromkeys(hosts))
        self.nodes = len(ordered_hosts)
        expected = [host for host in ordered_hosts for _ in range(self.world // self.nodes)]
        if hosts != expected:
            raise ValueError("WeftMoE requires equal-size, contiguous node-local EP teams")
        self.experts, self.top_k = experts, top_k
        self.hidden, self.intermediate = hidden, intermediate
        self.training = training
        self.decode_only = decode_only
        self.fp8_workspace = fp8_workspace
        self.precision = precision or ("fp8" if fp8_workspace else "bf16")
        self.max_tokens = max_tokens
        self.stream = stream
        if self.stream is None:
            self.stream = torch.cuda.current_stream() if training else torch.cuda.Stream()
        # Agree before any native collective: a bad shape on one rank must be a collective error,
        # not a peer stranded in the handle exchange (reference: weftmoe/runtime.py:83-105).
        request = dict(
            precision=self.precision, nvfp4_scales=nvfp4_scales, experts=experts, top_k=top_k,
            hidden=hidden, intermediate=intermediate, max_tokens=max_tokens, max_rows=max_rows,
            max_saved=max_saved, training=training, batch_invariant=batch_invariant,
            fp8_workspace=fp8_workspace, decode_only=decode_only, input_layout=input_layout,
        )
        requests = col.all_gather_object(request)
        if any(r != request for r in requests):
            raise ValueError("EP ranks requested incompatible WeftMoE configurations")
        if nvfp4_scales is not None and self.precision != "nvfp4":
            raise ValueError("nvfp4_scales requires NVFP4 precision")
        if self.nodes != 1:
            raise ValueError("This build serves one NVLink node: EP ranks must share a host")
        if self.precision not in ("bf16", "fp8", "nvfp4") or input_layout != "dp":
            raise ValueError("Unsupported runtime precision")
        if fp8_workspace and self.precision != "fp8":
            raise ValueError("Unsupported runtime precision")
        if self.precision == "nvfp4":
            from .nvfp4 import NVFP4Scales, _validate_scales
            if intermediate % 256:
                raise ValueError("NVFP4 requires intermediate divisible by 256")
            self.nvfp4_scales = NVFP4Scales() if nvfp4_scales is None else NVFP4Scales(*nvfp4_scales)
            _validate_scales(self.nvfp4_scales)
        if hidden > 4096 and hidden % 512:
            raise ValueError("Blackwell combine requires hidden divisible by 512 when hidden > 4096")
        if decode_only:
            # A decode runtime (reference: the DT runtime, docs/usage.md:104-112) serves inference only and
            # keeps every call within the single-launch route planner, so that a decode step is the same
            # short launch sequence whatever the batch.
            if training:
                raise ValueError("decode_only runtimes are inference-only (training=False)")
            if max_tokens * top_k > DECODE_MAX_ROUTES:
                raise ValueError(f"decode_only runtimes hold at most {DECODE_MAX_ROUTES} routes per rank "
                                 f"(max_tokens * top_k = {max_tokens * top_k})")
        if (max_tokens < 0 or hidden < 256 or hidden % 256 or not 128 <= intermediate <= 4096
                or intermediate % 128 or experts % self.world or not 1 <= top_k <= min(32, experts)
                or experts > 2048 or experts // self.world > 512
                or self.world not in (1, 2, 4, 8)):
            raise ValueError("Unsupported Blackwell expert shape or token capacity")
        factory = _native_factory or NativeRuntime
        extra = () if self.precision == "bf16" else (self.precision,)
        self.native = factory(col, experts, top_k, hidden, intermediate, max_tokens, max_rows,
                              self.stream, training, max_saved if training else 1, *extra)
        if self.precision == "nvfp4":
            self.native.scales = self.nvfp4_scales
        self.stream = getattr(self.native, "stream", self.stream)
        self.compilation = None

    def _check(self, x, routes, gates, w1, w2):
        if self.native is None:
            raise RuntimeError("WeftMoE runtime is closed")
        if self.precision == "fp8":
            raise ValueError("Compact FP8 workspace requires forward_fp8 or moe(..., fp8_weights=...)")
        if self.precision == "nvfp4" and not self.training:
            raise ValueError("NVFP4 inference runtimes take inference_nvfp4")
        if self.training and torch.cuda.current_stream() != self.stream:
            raise RuntimeError("Runtime must be invoked on its preparation stream")
        if x.ndim != 2 or x.shape[1] != self.hidden or x.shape[0] > self.max_tokens:
            raise ValueError("Activation shape exceeds prepared capacity")
        shapes = (
            (x.shape[0], self.top_k),
            (x.shape[0], self.top_k),
            (self.experts // self.world, 2 * self.intermediate, self.hidden),
            (self.experts // self.world, self.hidden, self.intermediate),
        )
        for tensor, shape in zip((routes, gates, w1, w2), shapes):
            if tensor.shape != shape:
                raise ValueError(f"Expected {shape}, got {tuple(tensor.shape)}")
        for tensor, dtype in zip((x, routes, gates, w1, w2),
                                 (torch.bfloat16, torch.int32, torch.float32, torch.bfloat16,
                                  torch.bfloat16)):
            if (tensor.dtype != dtype or tensor.device != x.device or not tensor.is_cuda
                    or not tensor.is_contiguous()):
                raise ValueError(f"Expected contiguous CUDA {dtype} on {x.device}")

    def forward(self, x, routes, gates, w1, w2):
        self._check(x, routes, gates, w1, w2)
        return self.native.forward(x, routes, gates, w1, w2)

    def forward_async(self, x, routes, gates, w1, w2, *, retain_backward_state=True):
        """Enqueue FWD, optionally omitting X/AB for checkpoint's no-grad pass."""
        self._check(x, routes, gates, w1, w2)
        return self.native.forward_async(x, routes, gates, w1, w2, retain_backward_state)

    def _check_fp8_source(self, source):
        """A prequantised source (x or dY): rows quantised 1 x 128 by quantize_fp8, one row per token."""
        if self.precision != "fp8":
            raise ValueError("Source must be BF16 or FP8Tensor with explicit row scales")
        if (len(source.shape) != 2 or source.block_rows != 1 or source.shape[1] != self.hidden
                or source.shape[0] > self.max_tokens or source.data.device != self.stream.device):
            raise ValueError("Source shape/device/layout does not match runtime")

    def _check_dy(self, dy):
        from .fp8 import FP8Tensor
        if isinstance(dy, FP8Tensor):
            return self._check_fp8_source(dy)
        if not isinstance(dy, torch.Tensor) or dy.dtype != torch.bfloat16:
            raise ValueError("Source must be BF16 or FP8Tensor with explicit row scales")
        if (dy.ndim != 2 or dy.shape[1] != self.hidden or dy.shape[0] > self.max_tokens
                or not dy.is_cuda or not dy.is_contiguous() or dy.device != self.stream.device):
            raise ValueError("Source shape/device/layout does not match runtime")

    def backward(self, tape, dy):
        """Consume BF16 dY; returns (dx, dgates, dw1, dw2)."""
        if torch.cuda.current_stream() != self.stream:
            raise RuntimeError("Backward must use the preparation stream")
        dy = dy.contiguous() if isinstance(dy, torch.Tensor) else dy
        self._check_dy(dy)
        return self.native.backward(tape, dy)

    def backward_async(self, tape, dy):
        """Return stream-ordered gradients without waiting."""
        if torch.cuda.current_stream() != self.stream:
            raise RuntimeError("Backward must use the preparation stream")
        dy = dy.contiguous() if isinstance(dy, torch.Tensor) else dy
        self._check_dy(dy)
        return self.native.backward_async(tape, dy)

    def _check_quantized(self, x, routes, gates):
        from .fp8 import FP8Tensor
        if self.native is None:
            raise RuntimeError("WeftMoE runtime is closed")
        if isinstance(x, FP8Tensor):
            self._check_fp8_source(x)
            x = x.data
        elif (not isinstance(x, torch.Tensor) or x.dtype != torch.bfloat16 or x.ndim != 2
                or x.shape[1] != self.hidden or x.shape[0] > self.max_tokens or not x.is_cuda
                or not x.is_contiguous() or x.device != self.stream.device):
            raise ValueError("Source shape/device/layout does not match runtime")
        for value, dtype in ((routes, torch.int32), (gates, torch.float32)):
            if (value.shape != (x.shape[0], self.top_k) or value.dtype != dtype or not value.is_cuda
                    or value.device != x.device or not value.is_contiguous()):
                raise ValueError(f"Expected contiguous CUDA {dtype} of shape {(x.shape[0], self.top_k)}")

    def _check_fp8_weights(self, weights, device):
        from .fp8 import PreparedFP8Weights
        if not isinstance(weights, PreparedFP8Weights):
            raise TypeError("weights must be PreparedFP8Weights")
        if (weights.w1.shape != (self.experts // self.world, 2 * self.intermediate, self.hidden)
                or weights.w2.shape != (self.experts // self.world, self.hidden, self.intermediate)
                or weights.w1.data.device != device):
            raise ValueError("Prepared FP8 weights do not match runtime shape/device")

    def forward_fp8(self, x, routes, gates, weights, *, synchronize=True,
                    retain_backward_state=True, weight_grad_dtype=torch.float32):
        """PF forward with BF16 input quantised online (1x128) and prepared FP8 weights.

        Prepare weights with weftmoe_b200.fp8.prepare_fp8_weights before this call (training=True when
        a backward pass will follow).  Backward runs dU and dX in FP8 and the two weight gradients in
        BF16 on the dequantised saved rows.  x (and dY in backward) may also be an FP8Tensor quantised
        1 x 128 by quantize_fp8: its bytes and scales are used as they are and give the same result bits as
        the BF16 source (reference: tests/torchrun_fp8.py:133-157)."""
        if weight_grad_dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("weight_grad_dtype must be torch.bfloat16 or torch.float32")
        if self.precision != "fp8":
            raise ValueError("Prepare an FP8 runtime first (precision='fp8' or fp8_workspace=True)")
        if self.training and torch.cuda.current_stream() != self.stream:
            raise RuntimeError("Runtime must be invoked on its preparation stream")
        self._check_quantized(x, routes, gates)
        self._check_fp8_weights(weights, getattr(x, "data", x).device)   # x: BF16 tensor or FP8Tensor
        weights.wait(training=self.training and retain_backward_state)
        return self.native.forward_fp8(x, routes, gates, weights, synchronize, retain_backward_state,
                                       weight_grad_dtype == torch.float32)

    def inference_fp8(self, layer, x, routes, gates, weights):
        """Replayable FP8 inference with stable input addresses (reference: weftmoe/runtime.py:387-415)."""
        if self.training or self.precision != "fp8":
            raise ValueError("inference_fp8 requires an FP8 runtime with training=False")
        self._check_quantized(x, routes, gates)
        self._check_fp8_weights(weights, getattr(x, "data", x).device)
        if torch.cuda.is_current_stream_capturing():
            weights._validate_version()
        else:
            weights.wait(training=False)
        return self.native.graph_forward(layer, x, routes, gates, weights.w1.data, weights.w2.data,
                                         torch.cuda.current_stream().cuda_stream, weights)

    def inference_nvfp4(self, layer, x, routes, gates, weights, *, x_scale=None, intermediate_scale=None):
        """Run prepared NVFP4 experts with online block-16 activation quantization."""
        from .nvfp4 import NVFP4Weights, _validate_scales
        if self.precision != "nvfp4" or self.training:
            raise ValueError("Prepare an NVFP4 inference runtime first")
        self._check_quantized(x, routes, gates)
        if not isinstance(weights, NVFP4Weights):
            raise TypeError("Expected prepared NVFP4 expert weights")
        e = self.experts // self.world
        if (weights.fc1[0].shape != (e, 2 * self.intermediate, self.hidden // 2)
                or weights.fc2[0].shape != (e, self.hidden, self.intermediate // 2)):
            raise ValueError("NVFP4 weights do not match the prepared experts")
        x_scale = self.nvfp4_scales.x if x_scale is None else x_scale
        intermediate_scale = self.nvfp4_scales.intermediate if intermediate_scale is None else intermediate_scale
        _validate_scales((x_scale, intermediate_scale))
        return self.native.inference(x, routes, gates, weights, x_scale, intermediate_scale)

    def drain(self):
        """Finish the pending training call before inspecting or releasing leases."""
        self.native.drain_training()

    def inference(self, layer, x, routes, gates, w1, w2):
        self._check(x, routes, gates, w1, w2)
        return self.native.graph_forward(layer, x, routes, gates, w1, w2,
                                         torch.cuda.current_stream().cuda_stream)

    def inference_eager(self, x, routes, gates, w1, w2, *, layer=None):
        """Run changing inputs/routes; `layer` is accepted for API compatibility."""
        self._check(x, routes, gates, w1, w2)
        return self.native.eager_inference(x, routes, gates, w1, w2,
                                           torch.cuda.current_stream().cuda_stream,
                                           *(() if layer is None else (layer,)))

    def inference_eager_async(self, x, routes, gates, w1, w2, *, layer=None):
        self._check(x, routes, gates, w1, w2)
        return self.native.eager_inference_async(x, routes, gates, w1, w2,
                                                 torch.cuda.current_stream().cuda_stream,
                                                 *(() if layer is None else (layer,)))

    def invalidate_inference_layer(self, layer):
        self.native.invalidate_inference_layer(layer, torch.cuda.current_stream().cuda_stream)

    def close(self):
        """Collectively release native CUDA/IPC storage at a phase boundary."""
        if self.native is None:
            return
        torch.cuda.synchronize()
        self.drain()
        self.native.drain_eager_inference()
        if self.training and self.native.usage()["notify_slots_in_use"]:
            raise RuntimeError("Live backward tapes prevent closing the runtime")
        self._collectives.barrier()
        self.native.retire_peer_mappings()
        # No exporter may free its storage while another rank still has an IPC import.
        self._collectives.barrier()
        if hasattr(self.native, "destroy"):
            self.native.destroy()
        self.native = None


class _MoE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, runtime, x, routes, gates, w1, w2):
        ctx.runtime = runtime
        ctx.tape = runtime.forward(x, routes, gates, w1, w2)
        return ctx.tape.output

    @staticmethod
    def backward(ctx, dy):
        dx, dg, dw1, dw2 = ctx.runtime.backward(ctx.tape, dy)
        ctx.tape = None
        ctx.runtime = None
        return None, dx, None, dg, dw1, dw2


class _MoEFP8(torch.autograd.Function):
    @staticmethod
    def forward(ctx, runtime, x, routes, gates, w1, w2, weights):
        if (w1.shape != weights.w1.shape or w2.shape != weights.w2.shape
                or w1.dtype not in (torch.bfloat16, torch.float32)
                or w2.dtype not in (torch.bfloat16, torch.float32)
                or w1.device != x.device or w2.device != x.device):
            raise ValueError("FP8 autograd requires matching BF16/FP32 parameter tensors")
        ctx.runtime = runtime
        ctx.save_for_backward(w1, w2)
        weights.validate_parameters(w1, w2)
        grad_dtype = torch.bfloat16 if w1.dtype == w2.dtype == torch.bfloat16 else torch.float32
        ctx.tape = runtime.forward_fp8(x, routes, gates, weights, weight_grad_dtype=grad_dtype)
        return ctx.tape.output

    @staticmethod
    def backward(ctx, dy):
        w1, w2 = ctx.saved_tensors  # detect optimizer updates before backward
        dx, dg, dw1, dw2 = ctx.runtime.backward(ctx.tape, dy)
        ctx.tape = None
        ctx.runtime = None
        return None, dx, None, dg, dw1.to(w1.dtype), dw2.to(w2.dtype), None


def moe(runtime, x, routes, gates, w1, w2, *, fp8_weights=None):
    """Apply the fused operation, preserving router and expert autograd edges."""
    if torch.is_grad_enabled() and not runtime.training:
        raise ValueError("Autograd requires a runtime prepared with training=True")
    if fp8_weights is not None:
        return _MoEFP8.apply(runtime, x, routes, gates, w1, w2, fp8_weights)
    return _MoE.apply(runtime, x, routes, gates, w1, w2)
