"""`lt.distributed`: process group, collectives, device mesh, FSDP / TP / SP / PP / CP / EP."""
from .process_group import (FileStore, OverlappedAllReducer, ProcessGroup, RankFailure, TCPStore, Watchdog,
                            all_gather, all_reduce, all_reduce_async, all_reduce_bucketed, all_reduce_grads, barrier,
                            broadcast, get_rank, get_world_size, init_process_group, overlapped_all_reduce,
                            overlapped_reduce_scatter, recv_tensor, reduce_scatter, send_tensor, shutdown,
                            sync_overlapped_all_reduce)
from .mesh import DeviceMesh, DTensor, Placement, PlacementType, distribute_tensor
from .tp import ColumnParallelLinear, RowParallelLinear, vocab_parallel_cross_entropy
from .pp import PipelineParallelModule
from .cp import (context_parallel_backward, context_parallel_forward, ring_attention, zigzag_merge, zigzag_positions,
                 zigzag_split)
from .ep import MoEFeedForward
from .ulysses import head_to_seq, seq_to_head, ulysses_attention
from .fsdp_api import FSDP, FullyShardedDataParallel


def __getattr__(name):
    # imported on first use, so that `python -m litetorch_b200.parallel.elastic` does not find its module half-loaded
    if name == "ElasticLauncher":
        from .elastic import ElasticLauncher
        return ElasticLauncher
    if name == "elastic":
        import importlib
        return importlib.import_module(".elastic", __name__)
    raise AttributeError("module %r has no attribute %r" % (__name__, name))
from ..core import manual_seed

__all__ = [n for n in dir() if not n.startswith("_")] + ["ElasticLauncher"]

# the reference's bindings export the enum values into the module as well (py::enum_::export_values,
# src/bindings/python_bindings.cpp:748-752)
SHARD, REPLICATE, PARTIAL = PlacementType.SHARD, PlacementType.REPLICATE, PlacementType.PARTIAL
