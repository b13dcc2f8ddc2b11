"""FX sub-graph -> the 6-tuple IR.  From-scratch equivalent of the reference tracer
(trace/graph_trace.py:32-328): it walks the nodes of a fused ``easier`` sub-module and classifies them
into inputs, outputs, selector registers, map operations, reducers and aggregators, producing dicts with
the same keys.  Selector / Reducer modules and node metadata come from the third-party ``easier``
package, which is imported lazily; ``trace_graph`` can also be driven with duck-typed stand-ins (tests):
``is_selector(node)``, ``is_reducer(node)`` and ``node_meta(node) -> (shape, dtype)`` callables.
"""
from __future__ import annotations

from typing import Any, Callable, Dict, List, Optional, Tuple

def classify_op(target: Any) -> str:
    """Name of the IR op for an FX call target; the substring tests and their order are the reference's
    (trace/graph_trace.py:229-276), including the leading blank in ' lt' / ' gt' / ' where' that only
    matches "<built-in function lt>"-style reprs."""
    t = str(target)
    if "add" in t and "add_" not in t:
        return "add"
    for frag, op in (("mul", "mul"), ("sub", "sub"), ("norm", "norm"), ("truediv", "truediv"), ("sum", "sum"),
                     ("neg", "neg"), ("add_", "add_"), ("pow", "pow"), ("setitem", "setitem"), ("getitem", "getitem"),
                     ("clone", "clone"), ("copy_", "copy_"), ("exp", "exp"), ("abs", "abs"), ("sign", "sign"),
                     (" lt", "lt"), (" gt", "gt"), (" where", "where")):
        if frag in t:
            return op
    raise ValueError(f"Operation {target} not supported")


def _easier_hooks(submodule, traced_model):
    from easier import Reducer, Selector                                    # third-party, absent in CI
    from easier.core.passes.dataflow_fusion.node_group import get_node_group
    from easier.core.runtime.metadata import get_node_meta
    group_nodes = {n.name: n for n in get_node_group(submodule).nodes}
    top_nodes = {n.name: n for n in traced_model.jit_engine.graph.nodes}

    def module_type(node):
        return list(group_nodes[node.name].meta["nn_module_stack"].values())[0][1]

    def meta(node):
        src = top_nodes if node.op == "placeholder" else group_nodes
        m = get_node_meta(src[node.name])
        return tuple(m.shape[1:]), m.dtype
    return (lambda n: n.op == "call_module" and module_type(n) == Selector,
            lambda n: n.op == "call_module" and module_type(n) == Reducer, meta)


def trace_graph(submodule, traced_model=None, is_selector: Optional[Callable] = None,
                is_reducer: Optional[Callable] = None, node_meta: Optional[Callable] = None):
    """Returns (inputs, outputs, selector_register, map_operations, reducer_operations,
    aggregator_operations)."""
    if is_selector is None or is_reducer is None or node_meta is None:
        is_selector, is_reducer, node_meta = _easier_hooks(submodule, traced_model)

    def info(node) -> Tuple[Tuple[int, ...], Any]:
        shape, dtype = node_meta(node)
        return (tuple(shape) if tuple(shape) != () else (1,)), dtype

    def clean(t):
        return t.replace(".", "_") if isinstance(t, str) else t

    def argnames(args):
        return [a.name if hasattr(a, "name") else a for a in args]

    nodes = list(submodule.graph.nodes)
    out_node = nodes[-1]
    body = nodes[:-1]
    out_args = out_node.args[0] if isinstance(out_node.args[0], (list, tuple)) else [out_node.args[0]]
    output_names = {a.name if hasattr(a, "name") else a for a in out_args}

    outputs: List[Dict[str, Any]] = []
    for n in out_args:
        shape, dtype = info(n)
        name, target, args = n.name, n.target, n.args
        if is_reducer(n):
            target = "reducer"
        elif n.op == "call_function" and "setitem" in str(target):
            name, target = args[0], args[-1]
        elif n.op == "call_function" and "sum" in str(target):
            target = "sum"
        outputs.append({"op": n.op, "name": name, "target": target, "dtype": "ValueT", "shape": shape,
                        "args": args, "dtype_data": dtype})

    selector_names = {n.name for n in body if is_selector(n)}
    selector_sources = {n.args[0].name for n in body if n.name in selector_names}

    inputs: List[Dict[str, Any]] = []
    for n in body:
        shape, dtype = info(n)
        if n.op == "placeholder" and n.name not in output_names:
            inputs.append({"name": n.name, "target": clean(n.target), "dtype": "scalar_t", "shape": shape, "op": n.op,
                           "args": n.args, "dtype_data": dtype})
        elif n.name in selector_names:
            inputs.append({"name": n.name, "target": clean(n.target), "dtype": "int", "shape": shape, "op": n.op,
                           "args": n.args, "dtype_data": dtype})

    selector_register: List[Dict[str, Any]] = []
    for n in body:
        shape, dtype = info(n)
        if n.op == "placeholder" and n.name not in selector_sources and n.name not in output_names:
            selector_register.append({"name": n.name, "target": n.target, "dtype": "TensorT", "selector": 0,
                                      "selector_name": n.name, "shape": shape, "dtype_data": dtype})
        if n.name in selector_names:
            selector_register.append({"name": n.name, "target": n.args[0].name, "dtype": "TensorKeyT", "selector": 1,
                                      "selector_name": clean(n.target), "shape": shape, "dtype_data": dtype})

    map_operations: List[Dict[str, Any]] = []
    reducer_operations: List[Dict[str, Any]] = []
    aggregator_operations: List[Dict[str, Any]] = []
    for n in body:
        shape, dtype = info(n)
        if n.op == "call_module" and n.name not in selector_names:
            entry = {"name": n.name, "target": n.target, "op": "reducer", "shape": shape, "dtype_data": dtype,
                     "args": argnames(n.args)}
            map_operations.append(entry)
            reducer_operations.append({k: v for k, v in entry.items() if k != "target"})
        elif n.op in ("call_function", "call_method"):
            op = classify_op(n.target)
            entry = {"name": n.name, "target": n.target, "op": op, "shape": shape, "dtype_data": dtype,
                     "args": argnames(n.args)}
            map_operations.append(entry)
            if op == "sum":
                aggregator_operations.append({"name": n.name, "op": "sum", "shape": shape, "dtype_data": dtype,
                                              "args": argnames(n.args)})
    return inputs, outputs, selector_register, map_operations, reducer_operations, aggregator_operations
