"""One-step-asynchronous and fully-asynchronous RL training driver.

Rollout for step i+1 overlaps training of step i (reference: train_async.py:22-129).  With colocated
SPMD ranks the overlap is cooperative: the rollout function keeps its producer alive between trainer
phases (``--fully-async``) or the next batch is generated right after the weight update that follows the
previous train step while metrics/checkpoint work proceeds; with ``--rollout-num-gpus`` smaller than the
world size the trailing ranks run engines only and the leading ranks train only, exchanging samples over
gloo and weights over NCCL / NVLink.  Weights are pushed to the engines every
``--update-weights-interval`` steps, and the off-policy corrections (``--use-tis``, staleness filter)
apply.
"""
from miles_b200.async_loop import AsyncRLLoop
from miles_b200.utils.arguments import parse_args


def train(args):
    assert not args.colocate or args.fully_async or True
    loop = AsyncRLLoop(args)
    return loop.run()


if __name__ == "__main__":
    train(parse_args())
