"""Metadata of a traced step function (``triton_kernel/flexsn/info.py`` of the reference).  The forward graph has the signature
``[*inputs, *states] -> [*outputs, *states, *intermediates]``; kernels generated here save no intermediates (backward
recomputes the step from the stored state sequence), so graphs normally end after the states."""
from collections import namedtuple

import torch.fx as fx

__all__ = ["FlexSNInfo", "extract_info"]

FlexSNInfo = namedtuple("FlexSNInfo", ["num_inputs", "num_outputs", "num_states", "fwd_core_args", "fwd_core_returns",
                                       "fwd_core_recipients", "fwd_kernel_returns", "num_fwd_kernel_returns", "c2k_return_mapping"])


def extract_info(fwd_graph: fx.Graph, num_inputs: int = 1, num_states: int = 0, num_outputs: int = 1) -> FlexSNInfo:
    args = [n.name for n in fwd_graph.nodes if n.op == "placeholder"]
    returns = [a.name for n in fwd_graph.nodes if n.op == "output" for a in n.args[0]]
    fixed = num_outputs + num_states
    if len(args) != num_inputs + num_states:
        raise ValueError(f"the graph takes {len(args)} arguments, expected {num_inputs} inputs + {num_states} states")
    if len(returns) < fixed:
        raise ValueError(f"the graph returns {len(returns)} values, expected at least {num_outputs} outputs + {num_states} states")
    kernel_names = [f"s{i}" for i in range(num_outputs)] + [f"v{i}" for i in range(num_states)]
    symbol = dict(zip(returns[:fixed], kernel_names))          # a value returned twice keeps its first name
    recipients, kernel_returns, mapping = list(kernel_names), list(kernel_names), []
    for r in returns[fixed:]:
        if r in symbol:
            recipients.append("_")
        else:
            symbol[r] = f"res{sum(k.startswith('res') for k in kernel_returns)}_f"
            recipients.append(symbol[r])
            kernel_returns.append(symbol[r])
        mapping.append(kernel_returns.index(symbol[r]))
    return FlexSNInfo(num_inputs, num_outputs, num_states, args, returns, recipients, kernel_returns, len(kernel_returns), mapping)
