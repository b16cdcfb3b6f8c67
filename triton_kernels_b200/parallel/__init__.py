"""Multi-GPU sharding of the block path on one NVLink/NVSwitch box.

Two shardings, both one process per GPU over torch.distributed:
  * batch data-parallel (`data_parallel`): images are independent, weights replicated, no
    collective on the forward path;
  * Ulysses sequence parallelism (`ulysses`): tokens sharded, one all-to-all on heads before
    attention and one after.
The reference has no multi-GPU code; these follow the benchmark's sharded configs.
"""
from triton_kernels_b200.parallel.data_parallel import shard_batch
from triton_kernels_b200.parallel.ulysses import SequenceParallel, shard_joint_sequence

__all__ = ["SequenceParallel", "shard_batch", "shard_joint_sequence"]
