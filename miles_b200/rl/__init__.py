"""Backend-agnostic RL mathematics: KL estimators, advantage estimators, policy/value/SFT losses.

Everything operates on *flat packed* tensors: the response-aligned tokens of all samples of a
micro-batch are concatenated into one 1-D tensor and a ``seg`` vector maps each token to its sample.
Reductions are segment sums, so there are no Python loops over samples on the hot path.
"""
from .kl import compute_approx_kl  # noqa: F401
from .advantages import (  # noqa: F401
    chunked_gae,
    vanilla_gae,
    compute_advantages_and_returns,
    whiten,
)
from .losses import policy_loss, value_loss, sft_loss, SegmentReducer  # noqa: F401
from .rewards import normalize_group_rewards  # noqa: F401
