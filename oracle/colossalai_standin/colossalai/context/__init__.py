import enum


class ParallelMode(enum.Enum):
    GLOBAL = "global"
    DATA = "data"
    PIPELINE = "pipe"
    TENSOR = "tensor"
    PARALLEL_1D = "1d"
