"""Per-GPU worker process (the role of energonai/worker.py:19-110): joins the tensor-parallel
process group, builds the model shard, then serves batches that the engine delivers over RPC.

Differences from the reference: the process group is plain torch.distributed (NCCL on GPUs, gloo
on CPU-only hosts, which is what the tests use) instead of colossalai.launch, the tensor-parallel
context is energonai_b200.tp, and only one pipeline stage exists."""
import os
import threading
from typing import Any, Callable

import torch
import torch.distributed as dist
import torch.distributed.rpc as trpc
import torch.multiprocessing as mp

from . import tp
from .pipe import Pipe
from .task import RemoteFailure, TaskEntry

_stop = threading.Event()


def _request_stop() -> None:
    _stop.set()


def rpc_options(master_host: str, rpc_port: int, disable_shm: bool):
    kw = {"_transports": ["uv"]} if disable_shm else {}
    return trpc.TensorPipeRpcBackendOptions(init_method=f"tcp://{master_host}:{rpc_port}", **kw)


class Worker:
    def __init__(self, rank: int, tp_world_size: int, pp_world_size: int, master_host: str, master_port: int,
                 rpc_port: int, n_proc_per_node: int, model_fn: Callable[..., torch.nn.Module], pipe_size: int = 1,
                 rpc_disable_shm: bool = True, **model_kwargs: Any) -> None:
        self.global_rank, self.world_size = rank, tp_world_size * pp_world_size
        use_cuda = torch.cuda.is_available()
        if use_cuda:
            torch.cuda.set_device(rank % n_proc_per_node)
        os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = master_host, str(master_port)
        dist.init_process_group("nccl" if use_cuda else "gloo", rank=rank, world_size=self.world_size)
        ctx = tp.init_tp(tp_world_size)
        self.device = torch.device("cuda", torch.cuda.current_device()) if use_cuda else torch.device("cpu")
        self.rpc_name = f"worker{rank}"
        # The RPC layer comes up before the model is built, so that a model_fn that raises can be
        # reported to the master instead of leaving it waiting for a peer that never joins.
        trpc.init_rpc(self.rpc_name, rank=rank + 1, world_size=self.world_size + 1,
                      rpc_backend_options=rpc_options(master_host, rpc_port, rpc_disable_shm))
        self.input_pipe = Pipe(f"m_to_{rank}", "master", self.rpc_name, max_size=pipe_size)
        self.output_pipe = Pipe(f"{rank}_to_m", self.rpc_name, "master")
        self.poisoned = None                           # set once the device reported a failed wait
        try:
            model = model_fn(**model_kwargs)
            self.model = model.cuda() if use_cuda else model
            if use_cuda and tp_world_size > 1:
                # the all-reduces of the row-parallel layers run in the library's own kernels over
                # NVLink peer memory; where the peers' memory cannot be mapped, NCCL carries them
                try:
                    ctx.enable_peer_exchange_for(self.model)
                except RuntimeError:
                    ctx.peer = None
        except Exception as exc:                       # noqa: BLE001 (sent to the master)
            self.output_pipe.send(RemoteFailure(rank, f"{type(exc).__name__}: {exc}"))
            _stop.wait(10.0)                           # the master tears the RPC layer down
            trpc.shutdown(graceful=False)
            return
        self.output_pipe.send(0)                       # announce: pipeline rank of this worker
        self._serve()

    def _to_device(self, x):
        if torch.is_tensor(x):
            return x.to(self.device, non_blocking=True)
        if isinstance(x, dict):
            return {k: self._to_device(v) for k, v in x.items()}
        if isinstance(x, (list, tuple)):
            return type(x)(self._to_device(v) for v in x)
        return x

    def _forward(self, inputs: Any) -> Any:
        inputs = self._to_device(inputs)
        if isinstance(inputs, (tuple, list)):
            return self.model(*inputs)
        if isinstance(inputs, dict):
            return self.model(**inputs)
        return self.model(inputs)

    def _health(self):
        """None, or why this worker must not serve any more.  The kernels' waits (on tensor-core
        pipelines and on the flags of tensor-parallel peers) are bounded: when one runs out, the
        kernel records it in a device status word and returns, and the outputs of that call, and
        the exchange buffers from then on, cannot be trusted.  A model may add its own check by
        exposing `health()` (None or a message)."""
        if self.device.type == "cuda":
            from .gemm import device_status
            code, where, block, detail = device_status(clear=True)
            if code != 0:
                return f"device status {code} (wait site {where}, block {block}, detail {detail})"
        probe = getattr(self.model, "health", None)
        return probe() if callable(probe) else None

    def _serve(self) -> None:
        try:
            while not _stop.is_set():
                try:
                    task: TaskEntry = self.input_pipe.recv(timeout=0.05)
                except RuntimeError:
                    continue
                try:
                    if self.poisoned is not None:
                        raise RuntimeError(f"worker {self.global_rank} stopped serving after: {self.poisoned}")
                    with torch.inference_mode():
                        out = self._forward(task.batch)
                    out = out.cpu() if torch.is_tensor(out) else out   # (synchronises the device)
                    self.poisoned = self._health()
                    if self.poisoned is not None:
                        raise RuntimeError(self.poisoned)
                except Exception as exc:                 # answer the batch with the error, keep serving
                    out = RemoteFailure(self.global_rank, f"{type(exc).__name__}: {exc}")
                self.output_pipe.send(TaskEntry(task.uids, out))
        finally:
            # captured generation steps hold collective kernels: release them before the groups go
            # (tearing a process group down under a live graph can block)
            if hasattr(self.model, "_decode_state"):
                self.model._decode_state = None
            if self.device.type == "cuda":
                torch.cuda.synchronize()
            trpc.shutdown()
            if dist.is_initialized():
                dist.destroy_process_group()


def launch_workers(tp_world_size: int, pp_world_size: int, master_host: str, master_port: int, rpc_port: int,
                   model_fn: Callable[..., torch.nn.Module], n_proc_per_node: int = 1, node_rank: int = 0,
                   pipe_size: int = 1, rpc_disable_shm: bool = True, **model_kwargs: Any):
    ctx = mp.get_context("spawn")
    procs = []
    for i in range(n_proc_per_node):
        rank = n_proc_per_node * node_rank + i
        p = ctx.Process(target=Worker, args=(rank, tp_world_size, pp_world_size, master_host, master_port, rpc_port,
                                             n_proc_per_node, model_fn, pipe_size, rpc_disable_shm), kwargs=model_kwargs)
        p.start()
        procs.append(p)
    return procs
