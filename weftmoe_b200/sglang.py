"""SGLang `FusedMoE.forward` adapter over `TensorRuntime`.

Entry point `install(batch_invariant=True)` follows the reference's `weftmoe/sglang.py:215`; the row
sharding / staging / scatter helpers do the jobs of `weftmoe/_sglang_kernels.py:21-99` and the layout logic
of `weftmoe/sglang.py:363-487`.  On CUDA tensors staging and scatter are one kernel each of
libweftmoe_b200.so (`wm_stage_inputs`, `wm_scatter_output`); the torch expressions below define the same
results and serve host tensors.  SGLang is imported lazily: the helpers work without it.

Differences from the reference that follow from this runtime: masked top-k entries (-1) are legal route
ids here, so sanitisation only zeroes their gates instead of substituting unused experts; one runtime serves
prefill and decode (no separate decode-only runtime), and FP8 serving uses `inference_fp8` / `forward_fp8`.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .runtime import TensorRuntime

_runtime = None
_stream = None
_graph_inputs = {}
_use_fp8 = False
_fp8_weights = {}


def sanitize_routes(ids: torch.Tensor, weights: torch.Tensor):
    """int32 routes and fp32 gates for the runtime: masked entries keep id -1 and get gate 0."""
    routes = ids.to(torch.int32).contiguous()
    gates = torch.where(routes >= 0, weights.to(torch.float32), torch.zeros((), device=weights.device))
    return routes, gates.contiguous()


def _native_ok(hidden_states, ids, weights):
    """The staging kernel reads BF16 rows in 16-byte words, int32/int64 ids and FP32 weights, unit column stride."""
    return (hidden_states.dtype == torch.bfloat16 and hidden_states.stride(1) == 1 and hidden_states.stride(0) % 8 == 0
            and hidden_states.shape[1] % 8 == 0 and hidden_states.data_ptr() % 16 == 0
            and ids.dtype in (torch.int32, torch.int64) and ids.stride(1) == 1
            and weights.dtype == torch.float32 and weights.stride(1) == 1)


def row_shard(tokens: int, world: int, rank: int):
    """Replicated rows are split evenly across ranks: (rows per rank, first row, valid rows of this rank)."""
    local = (tokens + world - 1) // world
    start = rank * local
    return local, start, max(0, min(local, tokens - start))


def stage_inputs(hidden_states, topk_ids, topk_weights, start, valid_rows, local_rows, out=None):
    """This rank's slice of replicated inputs, padded to `local_rows` with zero rows whose routes are -1.
    `out` = (x, routes, gates) buffers with stable addresses (CUDA-graph capture)."""
    hidden = hidden_states.shape[1]
    k = topk_ids.shape[1]
    if out is None:
        out = (hidden_states.new_empty((local_rows, hidden)),
               torch.empty((local_rows, k), dtype=torch.int32, device=hidden_states.device),
               torch.empty((local_rows, k), dtype=torch.float32, device=hidden_states.device))
    x, routes, gates = out
    if hidden_states.is_cuda and _native_ok(hidden_states, topk_ids, topk_weights):
        from . import _lib
        with torch.cuda.device(hidden_states.device):
            _lib.check(_lib.load().wm_stage_inputs(
                _lib.ptr(hidden_states), hidden_states.stride(0), _lib.ptr(topk_ids),
                int(topk_ids.dtype == torch.int64), topk_ids.stride(0), _lib.ptr(topk_weights),
                topk_weights.stride(0), start, valid_rows, local_rows, hidden, k, _lib.ptr(x), _lib.ptr(routes),
                _lib.ptr(gates), torch.cuda.current_stream().cuda_stream))
        return x, routes, gates
    x.zero_()
    routes.fill_(-1)
    gates.zero_()
    if valid_rows:
        r, g = sanitize_routes(topk_ids[start:start + valid_rows], topk_weights[start:start + valid_rows])
        x[:valid_rows].copy_(hidden_states[start:start + valid_rows])
        routes[:valid_rows].copy_(r)
        gates[:valid_rows].copy_(g)
    return x, routes, gates


def scatter_output(output, tokens, start, valid_rows):
    """Place this rank's rows into a zero [tokens, H] tensor; the model's tensor-parallel reduction then
    reassembles every row (reference: weftmoe/sglang.py:470-482)."""
    if output.is_cuda and output.dtype == torch.bfloat16 and output.is_contiguous() and output.shape[1] % 8 == 0:
        from . import _lib
        result = output.new_empty((tokens, output.shape[1]))
        with torch.cuda.device(output.device):
            _lib.check(_lib.load().wm_scatter_output(_lib.ptr(output), tokens, start, valid_rows, output.shape[1],
                                                     _lib.ptr(result), torch.cuda.current_stream().cuda_stream))
        return result
    result = output.new_zeros((tokens, output.shape[1]))
    result[start:start + valid_rows].copy_(output[:valid_rows])
    return result


def _prepare_runtime(layer, group, top_k, max_tokens, *, batch_invariant, decode_only=False):
    global _stream
    if _stream is None:
        _stream = torch.cuda.Stream()
    return TensorRuntime(group=group, experts=layer.num_experts, top_k=top_k, hidden=layer.hidden_size,
                         intermediate=layer.w2_weight.shape[-1], max_tokens=max_tokens,
                         max_rows=max_tokens * top_k * 2 + layer.num_local_experts * 128, training=False,
                         stream=_stream, decode_only=decode_only, fp8_workspace=_use_fp8,
                         batch_invariant=batch_invariant)


def install(batch_invariant: bool = True, fp8: bool = False):
    """Route every `FusedMoE.forward` of SGLang through the expert operator (EP = TP, expert TP = 1)."""
    global _use_fp8
    try:
        from sglang.srt.distributed import get_tp_group
        from sglang.srt.layers.moe.fused_moe_triton.layer import FusedMoE
        from sglang.srt.model_executor.cuda_graph_runner import get_is_capture_mode
        from sglang.srt.server_args import get_global_server_args
    except ImportError as exc:
        raise ImportError("weftmoe_b200.sglang.install() needs SGLang to be importable") from exc
    _use_fp8 = fp8

    def forward(layer, hidden_states, topk_output):
        global _runtime
        group = get_tp_group().device_group
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        if layer.moe_ep_size != world or layer.moe_tp_size != 1:
            raise ValueError("WeftMoE SGLang requires EP=TP and expert TP=1")
        if layer.w13_weight.dtype != torch.bfloat16 or layer.w2_weight.dtype != torch.bfloat16:
            raise ValueError("WeftMoE SGLang requires unquantized BF16 experts")
        tokens, hidden = hidden_states.shape
        if tokens == 0:
            return torch.empty_like(hidden_states)
        args = get_global_server_args()
        k = topk_output.topk_ids.shape[-1]
        if _runtime is None:
            capacity = max(args.chunked_prefill_size or 8192, args.max_prefill_tokens or 16384,
                           args.cuda_graph_max_bs or 1)
            _runtime = _prepare_runtime(layer, group, k, (capacity + world - 1) // world,
                                        batch_invariant=batch_invariant)
        local, start, valid = row_shard(tokens, world, rank)
        capturing = get_is_capture_mode()
        buffers = None
        if capturing:  # the captured graph binds these addresses
            buffers = _graph_inputs.setdefault(local, stage_inputs(
                hidden_states, topk_output.topk_ids, topk_output.topk_weights, start, valid, local))
        x, routes, gates = stage_inputs(hidden_states, topk_output.topk_ids, topk_output.topk_weights, start,
                                        valid, local, out=buffers)
        if _use_fp8:
            from .fp8 import prepare_fp8_weights
            prepared = _fp8_weights.get(layer.layer_id)
            if prepared is None:
                prepared = _fp8_weights[layer.layer_id] = prepare_fp8_weights(
                    layer.w13_weight, layer.w2_weight, training=False)
            output = (_runtime.inference_fp8(layer.layer_id, x, routes, gates, prepared) if capturing else
                      _runtime.forward_fp8(x, routes, gates, prepared, synchronize=False,
                                           retain_backward_state=False).output)
        elif capturing:
            output = _runtime.inference(layer.layer_id, x, routes, gates, layer.w13_weight, layer.w2_weight)
        else:
            output = _runtime.inference_eager_async(x, routes, gates, layer.w13_weight, layer.w2_weight,
                                                    layer=layer.layer_id)
        if not layer.reduce_results:
            return scatter_output(output, tokens, start, valid)
        gathered = hidden_states.new_empty((local * world, hidden))
        dist.all_gather_into_tensor(gathered, output, group=group)
        return gathered[:tokens]

    FusedMoE.forward = forward
    FusedMoE._weftmoe_batch_invariant = batch_invariant
