"""Multi-GPU sharding of the block path on one NVLink/NVSwitch box.

Two shardings, both one process per GPU over torch.distributed:
  * batch data-parallel (`data_parallel`): images are independent, weights replicated, no
    collective on the forward path;
  * Ulysses sequence parallelism (`ulysses`): tokens sharded, heads exchanged before attention
    and tokens after it, either as two NCCL all-to-alls or as stores into peer memory issued by
    the producing kernels (`peer`).
The reference has no multi-GPU code; these follow the benchmark's sharded configs.
"""
from triton_kernels_b200.parallel.data_parallel import shard_batch
from triton_kernels_b200.parallel.ulysses import SequenceParallel, peer_exchange_layout, shard_joint_sequence

__all__ = ["SequenceParallel", "peer_exchange_layout", "shard_batch", "shard_joint_sequence"]
