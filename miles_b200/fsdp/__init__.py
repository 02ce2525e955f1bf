"""Fully-sharded data-parallel trainer backend (``--train-backend fsdp``).

Pure data parallelism in which no rank keeps a whole copy of the model: every *unit* (the embedding, each decoder layer,
the head) is cut into equal shards over the ranks of the shard group, together with its fp32 master weights and Adam
moments. A unit's full parameters exist only while it computes: they are all-gathered into one of a few rotating
buffers just before the unit runs (the next unit's gather is issued while the current one computes, on a stream of its
own), and its gradients are reduce-scattered into the rank's fp32 gradient shard as soon as the backward has left the
unit. With ``--dp-replicate-size R`` the ranks form an ``R x (world / R)`` mesh: shards inside a replica, gradient
all-reduce between replicas (hybrid sharding).

The model code does not know about any of this: ``FsdpParamStore`` offers the same ``params`` / ``grads`` mappings as
``ParamStore`` and materialises a unit when one of its parameters is looked up.

Counterpart of the reference's FSDP2 backend (miles/backends/fsdp_utils/actor.py:54-761 ``apply_fsdp2``,
parallel.py:14-103 mesh, checkpoint.py:78-250, update_weight_utils.py:54-294), which wraps a HuggingFace module with
``fully_shard`` per decoder layer; here the same schedule runs over the flat parameter store of this package, so both the
autograd model path and the hand-written forward / backward of the sm_100a path train under it, and its checkpoints are
the same reshardable atom format as the other backend's (either backend loads what the other saved).
"""
from .mesh import FsdpMesh, build_mesh
from .store import FsdpParamStore, Unit, build_units

__all__ = ["FsdpMesh", "build_mesh", "FsdpParamStore", "Unit", "build_units"]
