"""Synchronous RL training driver (colocated trainer + rollout engine on every GPU).

    python train.py <flags>                                   # one GPU
    torchrun --nproc-per-node 8 train.py <flags>              # one process per GPU

Accepts the flag surface of the reference's ``train.py`` (see ``miles_b200/utils/arguments.py``).
Loop: generate -> [offload rollout] -> [critic train] -> actor train -> save -> [offload train] ->
update weights -> eval, as in the reference driver train.py:22-150.
"""
from miles_b200.loop import RLLoop
from miles_b200.utils.arguments import parse_args


def train(args):
    loop = RLLoop(args)
    return loop.run()


if __name__ == "__main__":
    train(parse_args())
