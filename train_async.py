"""One-step-asynchronous and fully-asynchronous RL training driver (reference: train_async.py:22-129).

* Engines in other processes (``--rollout-engine-urls`` or ``--launch-rollout-fleet``): the rollout of step i+1 is
  generated on a background thread while step i trains and is collected before the weights change.
* Colocated engine (one process per GPU, trainer and engine on the same device): the next batch is generated right
  after the weight update that follows a train step (with the newest weights, or with weights up to
  ``--update-weights-interval`` steps old); generation and training do not run at the same time on one GPU.
* ``--fully-async``: a persistent producer (``rollout/fully_async_rollout.py``) keeps groups in flight across steps; it
  is advanced once per step before training, and ``--pause-generation-mode in_place|retract`` decides what happens to
  requests in flight during a weight update.

Weights are pushed to the engines every ``--update-weights-interval`` steps; the off-policy corrections (``--use-tis``,
``--max-weight-staleness``) apply.
"""
from miles_b200.async_loop import AsyncRLLoop
from miles_b200.utils.arguments import parse_args


def train(args):
    loop = AsyncRLLoop(args)
    return loop.run()


if __name__ == "__main__":
    train(parse_args())
