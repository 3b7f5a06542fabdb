"""``make_backend``: the ``torch.compile`` backend of the drop-in surface.

Same options, defaults, validation messages and attributes as the reference's
``make_backend`` (src/megabake/frontend.py:297-330, 508-623).  What differs is what
"compiling" means: the reference lowers an arbitrary FX graph through its own planner
and code generator; this backend recognises the one graph family the hand-written
megakernel runs -- a Llama/Qwen2-style decoder whose attention is declared through
``megabake::kv_attention`` (decode) or ``megabake::attention`` (prefill) -- binds its
parameters to a :class:`~megabake_b200.runtime.DecoderKernel`, checks the kernel against
the captured graph on the example inputs (the reference's 2 % relative-L2 gate,
src/megabake/compiler.py:240-241), and returns a callable with Dynamo's flat-argument
convention.  Anything else raises :class:`CompilerError` before any device work
(``fallback="error"``) or goes to Inductor when the error is marked safe
(``fallback="inductor"``).  ``compile_kernel=False`` (or CPU inputs) returns the
captured graph itself: the reference path.
"""

from __future__ import annotations

import operator
import threading
import time
from dataclasses import dataclass, field
from pathlib import Path
from types import MappingProxyType
from typing import Any, Callable, Mapping, Sequence

import torch
import torch.nn.functional as F

from . import ops  # noqa: F401  (registers the ops the graphs call)
from .diagnostics import CompilerDiagnostic, CompilerError
from .synth import DecoderConfig

GATE_RELATIVE_L2 = 0.02


def gate_limit(layers: int) -> float:
    """Relative-L2 limit of the first-call correctness gate (kernel against the captured graph).

    The reference allows 2 % for whole-model launches and otherwise falls back to a
    teacher-forced per-region check (src/megabake/compiler.py:235-248).  There are no regions
    to check one by one here, and two bf16 evaluations of one deep decoder already differ by
    more than 2 %: at 24 layers x 2048 channels, eager PyTorch and this kernel each sit 4.3-4.6 %
    from an fp32 evaluation and 2.9 % from each other on a 64-token prompt (measured on a B200).
    The limit therefore grows with depth: 2 % up to 8 layers, a quarter of a percent per layer
    beyond.  A wrong kernel lands at 100 % and more."""
    return max(GATE_RELATIVE_L2, 0.0025 * layers)


def _validate_options(options: Mapping[str, Any]) -> dict[str, Any]:
    unknown = set(options) - {"mode", "fallback", "cache", "model_name", "dump_dir", "compile_kernel", "scheduler"}
    if unknown:
        raise TypeError(f"Unsupported backend options: {', '.join(sorted(unknown))}")
    mode = options.get("mode", "prefill")
    if mode not in {"prefill", "decode"}:
        raise ValueError(f"Unsupported mode {mode!r}; expected 'prefill' or 'decode'")
    fallback = options.get("fallback", "error")
    if fallback not in {"error", "inductor"}:
        raise ValueError(f"Unsupported fallback {fallback!r}; expected 'error' or 'inductor'")
    cache = options.get("cache", True)
    if not isinstance(cache, bool):
        raise TypeError("cache must be a boolean")
    model_name = options.get("model_name", "model")
    if not isinstance(model_name, str) or not model_name:
        raise TypeError("model_name must be a non-empty string")
    dump_dir = options.get("dump_dir")
    if dump_dir is not None and not isinstance(dump_dir, (str, Path)):
        raise TypeError("dump_dir must be a path or None")
    compile_kernel = options.get("compile_kernel", None)
    if compile_kernel not in {None, True, False}:
        raise TypeError("compile_kernel must be True, False, or None for automatic")
    scheduler = options.get("scheduler", "auto")
    if scheduler not in {"phase", "region-events", "auto"}:
        raise ValueError("scheduler must be 'phase', 'region-events', or 'auto'")
    return dict(mode=mode, fallback=fallback, cache=cache, model_name=model_name, dump_dir=dump_dir,
                compile_kernel=compile_kernel, scheduler=scheduler)


@dataclass
class CaptureContext:
    """What the backend knows about one captured graph (the reference's CaptureContext,
    src/megabake/frontend.py:41-73, reduced to the fields callers read)."""

    mode: str
    fallback: str
    input_order: list[str]
    output_count: int
    requirements: dict[str, Any] = field(default_factory=dict)
    graph: Any = None


@dataclass
class DecoderBinding:
    """A recognised decoder graph: which flat inputs are which."""

    config: DecoderConfig
    stateful: bool
    ids_index: int
    positions_index: int | None
    weight_indices: dict[str, int]           # Hugging Face parameter name -> flat input index
    inv_freq_index: int
    state_indices: list[tuple[int, int, int]]  # per layer: key cache, value cache, valid length
    capacity: int
    batch: int
    sequence: int
    mask_node: Any = None                     # prefill: FX node of the additive mask (None = no mask tensor)


def _fail(stage: str, message: str, *, safe: bool = True, requirement: str | None = None) -> CompilerError:
    return CompilerError(CompilerDiagnostic(stage, message, requirement=requirement), safe_for_fallback=safe)


def _is_target(node, *targets) -> bool:
    return isinstance(node, torch.fx.Node) and node.op == "call_function" and node.target in targets


_KV_OPS = (torch.ops.megabake.kv_attention, torch.ops.megabake.kv_attention.default)
_ATT_OPS = (torch.ops.megabake.attention, torch.ops.megabake.attention.default)


def recognise_decoder(graph_module: torch.fx.GraphModule, example_inputs: Sequence[Any], mode: str) -> DecoderBinding:
    """Match the captured graph against the decoder the megakernel implements and return
    the binding of its flat inputs; raise ``CompilerError`` (stage ``plan-search``) otherwise."""
    graph = graph_module.graph
    placeholders = [node for node in graph.nodes if node.op == "placeholder"]
    index_of = {node: position for position, node in enumerate(placeholders)}
    if len(placeholders) != len(example_inputs):
        raise _fail("plan-search", "placeholder count does not match the example inputs")

    def tensor(node):
        return example_inputs[index_of[node]]

    kv_nodes = [node for node in graph.nodes if _is_target(node, *_KV_OPS)]
    att_nodes = [node for node in graph.nodes if _is_target(node, *_ATT_OPS)]
    if kv_nodes and att_nodes:
        raise _fail("plan-search", "graph mixes stateful and stateless attention")
    if kv_nodes and mode == "prefill":
        raise ValueError("prefill mode cannot compile a stateful KV cache update")
    attention_nodes = kv_nodes or att_nodes
    if not attention_nodes:
        raise _fail("plan-search", "no megabake::kv_attention or megabake::attention call in the graph",
                    requirement="declare attention through the megabake ops (attn_implementation='megabake')")
    stateful = bool(kv_nodes)
    layers = len(attention_nodes)

    embeddings = [node for node in graph.nodes if _is_target(node, F.embedding)]
    if len(embeddings) != 1 or embeddings[0].args[0] not in index_of or embeddings[0].args[1] not in index_of:
        raise _fail("plan-search", "expected one token-embedding gather fed by graph inputs")
    ids_node, embed_node = embeddings[0].args[0], embeddings[0].args[1]

    linears = [node for node in graph.nodes if _is_target(node, F.linear)]
    if len(linears) != 7 * layers + 1:
        raise _fail("plan-search", f"expected {7 * layers + 1} linear projections for {layers} layers, found {len(linears)}")
    for node in linears:
        if node.args[1] not in index_of:
            raise _fail("plan-search", f"projection {node.name} does not take a parameter as its weight")

    def weight_and_bias(node):
        bias = node.args[2] if len(node.args) > 2 else node.kwargs.get("bias")
        return node.args[1], bias

    def norm_weight(node):
        """``weight * normalised.to(dtype)``: the placeholder operand of the multiply feeding a projection."""
        source = node.args[0]
        while _is_target(source, operator.getitem) and isinstance(source.args[0], torch.fx.Node):
            source = source.args[0]  # transformers slices the positions whose logits are kept
        if not _is_target(source, operator.mul):
            raise _fail("plan-search", f"projection {node.name} is not fed by an RMSNorm weight multiply")
        for operand in source.args:
            if operand in index_of:
                return operand
        raise _fail("plan-search", f"no norm weight found for {node.name}")

    eps_values = set()
    for node in graph.nodes:
        if _is_target(node, torch.rsqrt) and _is_target(node.args[0], operator.add):
            for operand in node.args[0].args:
                if isinstance(operand, float):
                    eps_values.add(operand)
    if len(eps_values) != 1:
        raise _fail("plan-search", f"expected one RMSNorm epsilon, found {sorted(eps_values)}")

    weights: dict[str, int] = {"model.embed_tokens.weight": index_of[embed_node]}
    has_bias = False
    for layer in range(layers):
        group = linears[7 * layer: 7 * layer + 7]
        q, k, v, o, first, second, down = group
        gate, up = (first, second) if any(_is_target(user, F.silu) for user in first.users) else (second, first)
        prefix = f"model.layers.{layer}."
        weights[prefix + "input_layernorm.weight"] = index_of[norm_weight(q)]
        weights[prefix + "post_attention_layernorm.weight"] = index_of[norm_weight(gate)]
        for name, node in (("self_attn.q_proj", q), ("self_attn.k_proj", k), ("self_attn.v_proj", v),
                           ("self_attn.o_proj", o), ("mlp.gate_proj", gate), ("mlp.up_proj", up),
                           ("mlp.down_proj", down)):
            weight, bias = weight_and_bias(node)
            weights[prefix + name + ".weight"] = index_of[weight]
            if bias is not None:
                if name.startswith("mlp") or name.endswith("o_proj") or bias not in index_of:
                    raise _fail("plan-search", f"unsupported bias on {prefix + name}")
                weights[prefix + name + ".bias"] = index_of[bias]
                has_bias = True
    head = linears[-1]
    returned = next(node for node in graph.nodes if node.op == "output").args[0]
    returned = list(returned) if isinstance(returned, (tuple, list)) else [returned]
    if len(returned) != 1 or returned[0] is not head:
        raise _fail("plan-search", f"the graph returns {len(returned)} values; the kernel returns the logits only",
                    requirement="return the lm_head output alone (call the model with use_cache=False)", safe=True)
    weights["model.norm.weight"] = index_of[norm_weight(head)]
    weights["lm_head.weight"] = index_of[head.args[1]]

    inv_freq = [node for node in placeholders if "inv_freq" in node.name]
    if len(inv_freq) != 1:
        raise _fail("plan-search", "expected one rotary inv_freq buffer among the graph inputs")

    embed = tensor(embed_node)
    q_weight = example_inputs[weights["model.layers.0.self_attn.q_proj.weight"]]
    k_weight = example_inputs[weights["model.layers.0.self_attn.k_proj.weight"]]
    gate_weight = example_inputs[weights["model.layers.0.mlp.gate_proj.weight"]]
    first_attention = attention_nodes[0]
    query_value = first_attention.args[0].meta.get("example_value")
    if query_value is None:
        raise _fail("plan-search", "attention operand carries no shape information")
    head_dim = int(query_value.shape[-1])
    if embed.dtype != torch.bfloat16:
        raise _fail("plan-search", f"the megakernel computes in bfloat16, the graph holds {embed.dtype} parameters")
    rope_style = "hf" if any(_is_target(node, operator.neg) for node in graph.nodes) else "half_swap"
    config = DecoderConfig(
        hidden=int(embed.shape[1]), layers=layers, q_heads=int(q_weight.shape[0]) // head_dim,
        kv_heads=int(k_weight.shape[0]) // head_dim, head_dim=head_dim, intermediate=int(gate_weight.shape[0]),
        vocab=int(embed.shape[0]), rms_eps=float(next(iter(eps_values))), qkv_bias=has_bias,
        tied=weights["lm_head.weight"] == weights["model.embed_tokens.weight"], rope_style=rope_style,
        name="captured",
    )
    ids = tensor(ids_node)
    if ids.dim() != 2 or ids.dtype != torch.int64:
        raise _fail("plan-search", "token ids must be an int64 [batch, sequence] graph input")
    integer_inputs = [node for node in placeholders
                      if node is not ids_node and isinstance(tensor(node), torch.Tensor)
                      and tensor(node).dtype in (torch.int64, torch.int32) and tensor(node).shape == ids.shape]
    positions_index = index_of[integer_inputs[0]] if integer_inputs else None

    state: list[tuple[int, int, int]] = []
    capacity = 0
    mask_node = None
    if stateful:
        if ids.shape[1] != 1:
            raise _fail("plan-search", "megabake kv_attention supports one-token decode only")
        if positions_index is None:
            raise _fail("plan-search", "a decode graph needs position ids as an input")
        for node in attention_nodes:
            triple = node.args[3:6]
            if any(operand not in index_of for operand in triple):
                raise _fail("plan-search", "KV state must be passed as graph inputs")
            state.append(tuple(index_of[operand] for operand in triple))
        capacity = int(example_inputs[state[0][0]].shape[1])
    else:
        def mask_root(node):
            operand = node.args[3] if len(node.args) > 3 else None
            while _is_target(operand, operator.getitem) and isinstance(operand.args[0], torch.fx.Node):
                operand = operand.args[0]  # each layer cuts the shared mask to its key length
            return operand

        mask_node = first_attention.args[3] if len(first_attention.args) > 3 else None
        for node in attention_nodes[1:]:
            if mask_root(node) is not mask_root(first_attention):
                raise _fail("plan-search", "layers use different attention masks")
    return DecoderBinding(
        config=config, stateful=stateful, ids_index=index_of[ids_node], positions_index=positions_index,
        weight_indices=weights, inv_freq_index=index_of[inv_freq[0]], state_indices=state, capacity=capacity,
        batch=int(ids.shape[0]), sequence=int(ids.shape[1]), mask_node=mask_node,
    )


def _slice_graph(graph_module: torch.fx.GraphModule, target) -> torch.fx.GraphModule:
    """A graph module with the same placeholders that computes only ``target``."""
    needed = set()
    stack = [target]
    while stack:
        node = stack.pop()
        if node in needed:
            continue
        needed.add(node)
        stack.extend(node.all_input_nodes)
    new_graph = torch.fx.Graph()
    remap: dict = {}
    for node in graph_module.graph.nodes:
        if node.op == "placeholder" or node in needed:
            remap[node] = new_graph.node_copy(node, lambda old: remap[old])
    new_graph.output(remap[target])
    return torch.fx.GraphModule(graph_module, new_graph)


def _tables_from_inv_freq(inv_freq: torch.Tensor, positions: int, device) -> tuple[torch.Tensor, torch.Tensor]:
    """cos/sin tables the way transformers' rotary embedding computes them from its buffer."""
    freqs = torch.arange(positions, dtype=torch.int64).to(torch.float32)[:, None] * inv_freq.detach().cpu().float()[None, :]
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos().to(torch.bfloat16).to(device).contiguous(), emb.sin().to(torch.bfloat16).to(device).contiguous()


def compile_decoder(graph_module, example_inputs, binding: DecoderBinding, context: CaptureContext) -> Callable[..., Any]:
    """Bind the recognised graph to the megakernel, gate it against the graph itself, and
    return the flat-argument callable."""
    from .runtime import DecoderKernel

    started = time.perf_counter()
    config = binding.config
    device = example_inputs[binding.ids_index].device
    tokens = binding.batch * binding.sequence
    positions = binding.capacity if binding.stateful else max(binding.sequence, 16)
    weights = {name: example_inputs[index] for name, index in binding.weight_indices.items()}
    tables = _tables_from_inv_freq(example_inputs[binding.inv_freq_index], positions, device)
    try:
        kernel = DecoderKernel(config, weights, max_tokens=tokens, max_positions=positions, device=device, tables=tables)
    except CompilerError:
        raise
    mask_module = _slice_graph(graph_module, binding.mask_node) if binding.mask_node is not None else None
    lock = threading.Lock()
    weight_order = list(binding.weight_indices.items())
    bound_pointers = [tuple(example_inputs[index].data_ptr() for _, index in weight_order)]

    def forward(*args: Any, **kwargs: Any):
        if kwargs:
            raise TypeError(f"Unexpected keyword arguments: {', '.join(sorted(kwargs))}")
        if len(args) != len(example_inputs):
            raise CompilerError(CompilerDiagnostic(
                "input-binding", f"expected {len(example_inputs)} flat arguments, got {len(args)}"))
        with lock:
            pointers = tuple(args[index].data_ptr() for _, index in weight_order)
            if pointers != bound_pointers[0]:  # a parameter tensor was replaced: bind again by pointer
                kernel.bind({name: args[index] for name, index in weight_order})
                bound_pointers[0] = pointers
            ids = args[binding.ids_index]
            if binding.stateful:
                keys = [args[k] for k, _, _ in binding.state_indices]
                values = [args[v] for _, v, _ in binding.state_indices]
                lengths = [args[n] for _, _, n in binding.state_indices]
                logits = kernel.decode(ids, args[binding.positions_index].to(torch.int64), keys, values, lengths)
            else:
                position_ids = None if binding.positions_index is None else args[binding.positions_index].to(torch.int64)
                mask = None
                if mask_module is not None:
                    with torch.no_grad():
                        mask = mask_module(*args)
                    mask = mask.expand(ids.shape[0], 1, ids.shape[1], ids.shape[1]).to(torch.bfloat16).contiguous()
                logits = kernel.prefill(ids, position_ids, mask)
        return (logits,) if context.output_count == 1 and context.requirements.get("tuple_output") else logits

    # Correctness gate on private copies of the state: the kernel against the captured graph.
    def private(value):
        return value.clone() if isinstance(value, torch.Tensor) else value

    state_positions = {index for triple in binding.state_indices for index in triple}
    reference_args = [private(v) if i in state_positions else v for i, v in enumerate(example_inputs)]
    kernel_args = [private(v) if i in state_positions else v for i, v in enumerate(example_inputs)]
    with torch.no_grad():
        expected = graph_module(*reference_args)
        actual = forward(*kernel_args)
    kernel.check()
    expected_tensor = expected[0] if isinstance(expected, (tuple, list)) else expected
    actual_tensor = actual[0] if isinstance(actual, (tuple, list)) else actual
    distance = float((actual_tensor.float() - expected_tensor.float()).norm() / expected_tensor.float().norm().clamp_min(1e-12))
    limit = gate_limit(config.layers)
    if not distance <= limit:
        raise _fail("correctness-gate", f"kernel output is {distance:.3g} in relative L2 from the captured graph "
                    f"(limit {limit:.3g})", safe=True)
    for triple in binding.state_indices:
        if int(kernel_args[triple[2]].item()) != int(reference_args[triple[2]].item()):
            raise _fail("correctness-gate", "valid length differs from the captured graph after one call")
    context.requirements.update(execution="megakernel", gate_relative_l2=distance)
    forward.megabake_compiled = kernel
    forward.megabake_runtime_state = kernel
    forward.megabake_context = context
    forward.megabake_trace = []
    forward.megabake_compile_us = (time.perf_counter() - started) * 1e6
    forward.megabake_cache_hit = False
    return forward


def _can_auto_compile(example_inputs: Sequence[Any]) -> bool:
    tensors = [value for value in example_inputs if isinstance(value, torch.Tensor)]
    if not tensors or any(value.device.type != "cuda" for value in tensors):
        return False
    try:
        return torch.cuda.get_device_capability(tensors[0].device) in {(10, 0), (10, 3)}
    except Exception:
        return False


def make_backend(**options: Any) -> Callable[..., Any]:
    """Backend for ``torch.compile(model, backend=make_backend(mode=...), fullgraph=True)``."""
    validated = _validate_options(options)
    contexts: list[CaptureContext] = []
    cache: dict[str, Any] = {}

    def backend(graph_module, example_inputs: Sequence[Any], **dynamo_kwargs: Any) -> Callable[..., Any]:
        if dynamo_kwargs:
            raise TypeError(f"Unsupported Dynamo backend options: {', '.join(sorted(dynamo_kwargs))}")
        if torch.is_grad_enabled() and any(isinstance(v, torch.Tensor) and v.requires_grad for v in example_inputs):
            raise RuntimeError("MegaBake supports inference only")
        if any(isinstance(v, torch.SymInt) for v in example_inputs):
            raise ValueError("symbolic shapes are not supported; compile with dynamic=False")
        placeholders = [node.name for node in graph_module.graph.nodes if node.op == "placeholder"]
        output_node = next(node for node in graph_module.graph.nodes if node.op == "output")
        returned = output_node.args[0]
        context = CaptureContext(
            mode=validated["mode"], fallback=validated["fallback"], input_order=placeholders,
            output_count=len(returned) if isinstance(returned, (tuple, list)) else 1,
            requirements={"inference_only": True, "execution": "reference",
                          "tuple_output": isinstance(returned, (tuple, list))},
            graph=graph_module,
        )
        contexts.append(context)
        backend.megabake_last_prepared = context
        backend.megabake_last_fallback = None
        compile_kernel = validated["compile_kernel"]
        wanted = compile_kernel is True or (compile_kernel is None and _can_auto_compile(example_inputs))
        forward = graph_module.forward
        if wanted:
            backend.megabake_last_compiled = backend.megabake_last_callable = None
            try:
                binding = recognise_decoder(graph_module, example_inputs, validated["mode"])
                if example_inputs[binding.ids_index].device.type != "cuda":
                    raise _fail("runtime-binding", "the megakernel runs on CUDA tensors only", safe=True)
                forward = compile_decoder(graph_module, example_inputs, binding, context)
                backend.megabake_last_compiled = forward.megabake_compiled
                backend.megabake_last_compile_us = forward.megabake_compile_us
                backend.megabake_last_trace = forward.megabake_trace
                backend.megabake_last_callable = forward
            except CompilerError as error:
                if validated["fallback"] != "inductor" or not error.safe_for_fallback:
                    raise
                from torch._inductor.compile_fx import compile_fx

                forward = compile_fx(graph_module, list(example_inputs))
                context.requirements.update(execution="inductor_fallback", fallback_reason=str(error))
                backend.megabake_last_fallback = forward
        elif validated["mode"] == "prefill" and any(_is_target(n, *_KV_OPS) for n in graph_module.graph.nodes):
            raise ValueError("prefill mode cannot compile a stateful KV cache update")
        try:
            forward.megabake_contexts = contexts
            forward.megabake_cache = cache
            forward.megabake_plan_cache = cache if validated["cache"] else None
        except AttributeError:  # bound methods take no attributes
            pass
        return forward

    backend.megabake_cache = cache
    backend.megabake_plan_cache = cache if validated["cache"] else None
    backend.megabake_contexts = contexts
    backend.megabake_options = MappingProxyType(validated)
    backend.megabake_prepare = lambda graph, inputs, **_: recognise_decoder(graph, inputs, validated["mode"])
    backend.megabake_last_prepared = backend.megabake_last_compiled = backend.megabake_last_callable = None
    backend.megabake_last_compile_us = backend.megabake_last_trace = backend.megabake_last_fallback = None
    backend.__name__ = "megabake_backend"
    return backend
