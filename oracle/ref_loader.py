"""Import the reference's own Python layer code on CPU (test infrastructure).

Works only where a checkout of the reference is present (environment variable
ENERGONAI_REFERENCE, default: a directory named `reference` beside this repository) and uses
the colossalai stand-in next to this file.  Returns None when the checkout is absent, so
callers can skip.
"""
import importlib
import os
import sys

_HERE = os.path.dirname(os.path.abspath(__file__))


def reference_root():
    root = os.environ.get("ENERGONAI_REFERENCE",
                          os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference"))
    return root if os.path.isdir(os.path.join(root, "energonai", "model")) else None


def load_reference_model_package():
    """Returns the imported `energonai.model` package of the reference, or None."""
    root = reference_root()
    if root is None:
        return None
    for p in (os.path.join(_HERE, "colossalai_standin"), root):
        if p not in sys.path:
            sys.path.insert(0, p)
    import torch
    # PipelineModel.forward builds the appended mask column on torch.cuda.current_device()
    # (model_factory.py:137-138); on a CPU-only run that has to resolve to the CPU.
    if not torch.cuda.is_available():
        torch.cuda.current_device = lambda: torch.device("cpu")
    return importlib.import_module("energonai.model")
