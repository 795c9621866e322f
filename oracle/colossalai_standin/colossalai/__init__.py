"""Stand-in for the third-party `colossalai` package (test infrastructure only).

The reference's model files import a handful of colossalai symbols (Linear1D_Col,
Linear1D_Row, LayerNorm1D, global_context, ...).  colossalai itself is not installable
offline, so this package restates the tensor-parallel-size-1 behaviour of exactly those
symbols over plain torch.nn, which lets the reference's own `energonai/model/*.py` run
unchanged on CPU to generate golden vectors.  Nothing in the product imports this.
"""


def launch(config=None, rank=0, world_size=1, host=None, port=None, backend=None, **kwargs):
    from .core import global_context
    global_context._launched = True
