"""The public surface of the installed reference package (``baseline/_ref/spikingjelly``), read as source text, against this
package: every module path resolves, every public top-level class / function exists under the same name, every public method
of a same-named class exists, and positional parameters come in the same order.  Skipped when the reference is not installed.

Known, intended differences are listed in ``DIFFERENT_SIGNATURES`` with the reason."""
import ast
import importlib
import inspect
import warnings
from pathlib import Path

import pytest

REF = Path(__file__).resolve().parents[1] / "baseline" / "_ref" / "spikingjelly"
pytestmark = pytest.mark.skipif(not REF.is_dir(), reason="reference package not installed under baseline/_ref")

# reason -> qualified names (suffix match)
DIFFERENT_SIGNATURES = {
    "a surrogate object is passed where the reference passes an id into its CuPy code registry": (
        "cupy_multistep_if_forward", "cupy_multistep_if_backward", "cupy_multistep_lif_forward", "cupy_multistep_lif_backward",
        "cupy_multistep_plif_forward", "cupy_multistep_plif_backward", "cupy_multistep_qif_forward", "cupy_multistep_eif_forward",
        "cupy_multistep_izhikevich_forward", "cupy_single_step_if_forward", "cupy_single_step_lif_forward", "NeuronBPKernel.__init__",
        "LIFNodeBPKernel.__init__"),
    "the CUDA generator works from traced graphs, not from a Triton code string": (
        "get_flexsn_inference_kernel", "get_flexsn_inference_final_state_kernel", "get_flexsn_forward_kernel", "get_flexsn_backward_kernel"),
    "internal node type of the auto_cuda generator, redesigned": ("VarNode.__init__",),
}
_ALLOWED = tuple(n for names in DIFFERENT_SIGNATURES.values() for n in names)


def _modules():
    for path in sorted(REF.rglob("*.py")):
        rel = path.relative_to(REF).with_suffix("")
        parts = list(rel.parts)
        if "examples" in parts:
            continue
        if parts[-1] == "__init__":
            parts = parts[:-1]
        yield ".".join(["spikingjelly_b200", *parts]), ast.parse(path.read_text())


def _positional(fn: ast.FunctionDef):
    return [a.arg for a in fn.args.posonlyargs + fn.args.args if a.arg not in ("self", "cls")]


def test_every_reference_module_and_public_name_has_a_counterpart():
    warnings.simplefilter("ignore")
    missing_modules, missing_names, missing_methods = [], [], []
    for name, tree in _modules():
        public = [n for n in tree.body if isinstance(n, (ast.ClassDef, ast.FunctionDef)) and not n.name.startswith("_")]
        if not public:
            continue
        try:
            mod = importlib.import_module(name)
        except ImportError as exc:
            missing_modules.append(f"{name}: {exc}")
            continue
        for node in public:
            if not hasattr(mod, node.name):
                missing_names.append(f"{name}.{node.name}")
            elif isinstance(node, ast.ClassDef):
                cls = getattr(mod, node.name)
                for m in node.body:
                    if isinstance(m, ast.FunctionDef) and not m.name.startswith("_") and not hasattr(cls, m.name):
                        missing_methods.append(f"{name}.{node.name}.{m.name}")
    assert not missing_modules, missing_modules
    assert not missing_names, missing_names
    assert not missing_methods, missing_methods


def test_positional_parameters_come_in_the_reference_order():
    warnings.simplefilter("ignore")
    differing = []
    for name, tree in _modules():
        try:
            mod = importlib.import_module(name)
        except ImportError:
            continue
        pairs = []
        for node in tree.body:
            if isinstance(node, ast.FunctionDef) and not node.name.startswith("_") and hasattr(mod, node.name):
                pairs.append((node.name, node, getattr(mod, node.name)))
            elif isinstance(node, ast.ClassDef) and not node.name.startswith("_") and hasattr(mod, node.name):
                cls = getattr(mod, node.name)
                for m in node.body:
                    if isinstance(m, ast.FunctionDef) and (m.name == "__init__" or not m.name.startswith("_")) and hasattr(cls, m.name):
                        pairs.append((f"{node.name}.{m.name}", m, getattr(cls, m.name)))
        for label, node, obj in pairs:
            try:
                params = inspect.signature(obj).parameters.values()
            except (TypeError, ValueError):
                continue
            if any(p.kind is p.VAR_POSITIONAL for p in params):
                continue
            ours = [p.name for p in params if p.kind in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD) and p.name not in ("self", "cls")]
            want = _positional(node)
            k = min(len(want), len(ours))
            if want[:k] != ours[:k] and not label.endswith(_ALLOWED):
                differing.append(f"{name}.{label}: reference {want} / here {ours}")
    assert not differing, "\n".join(differing)
