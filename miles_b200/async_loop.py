"""Asynchronous RL loop: rollout of step i+1 is produced while step i trains.

Two modes, selected like in the reference (train_async.py:22-129, miles/utils/arguments.py:3591-3609):

* one-step-async: generation of the next batch is started before the current batch is trained; the
  in-flight generation is drained before every weight update (every ``--update-weights-interval`` steps)
  so that engines are paused only for the sync window.
* ``--fully-async``: a persistent producer (``rollout.fully_async_rollout``) keeps groups in flight; the
  weight update uses ``--pause-generation-mode in_place|retract`` so that in-flight requests survive and
  record mixed weight versions; stale groups are filtered by ``--max-weight-staleness``.

With engines in other processes (``--rollout-engine-urls`` / ``--launch-rollout-fleet``) the next rollout is generated
on a background thread while the current one trains, and is collected before the weights change.

On one process per GPU the fully-asynchronous producer is advanced cooperatively: ``pump`` is called once per step
before training (engine iterations and training kernels do not interleave on one device); samples generated under
older weights are corrected by TIS when enabled.
"""
from __future__ import annotations

import time

from .loop import RLLoop
from .rollout.base_types import RolloutFnTrainInput
from .rollout.train_data import compute_rollout_metrics, flatten_groups, postprocess_rollout_data
from .utils.misc import should_run_periodic_action


def validate_async_off_policy_correction(args) -> None:
    """Async training is off-policy by construction: require an explicit correction or acknowledgement."""
    if getattr(args, "fully_async", False) and not (args.use_tis or args.use_rollout_logprobs or
                                                    getattr(args, "max_weight_staleness", None) is not None):
        print("[miles_b200] warning: --fully-async without --use-tis / --max-weight-staleness trains on stale samples uncorrected")


class AsyncRLLoop(RLLoop):
    def __init__(self, args, ps=None):
        validate_async_off_policy_correction(args)
        # the async drivers never release the KV cache between phases: engines keep generating
        args.offload_rollout = False
        super().__init__(args, ps)
        self._prefetched = None
        self._bg = None  # (thread, result box) of a generation that runs while the trainer trains (remote engines only)

    # ------------------------------------------------------------------ overlap with engines in other processes
    def _start_background_generation(self, rollout_id: int) -> None:
        import threading

        box: dict = {}

        def run():
            try:
                box["out"] = self._generate_now(rollout_id)
            except BaseException as e:  # surfaces in the training thread when the result is collected
                box["err"] = e

        th = threading.Thread(target=run, daemon=True)
        th.start()
        self._bg = (th, box)

    def _collect_background_generation(self):
        th, box = self._bg
        self._bg = None
        th.join()
        if "err" in box:
            raise box["err"]
        return box["out"]

    def _generate_now(self, rollout_id: int):
        t0 = time.perf_counter()
        out = self.rollout_fn(RolloutFnTrainInput(rollout_id))
        import asyncio

        if asyncio.iscoroutine(out):
            out = asyncio.run(out)
        if self.engine is not None and not getattr(self.args, "fully_async", False):
            self.engine.drain()
        samples = postprocess_rollout_data(self.local_args, flatten_groups(out.samples))
        m = dict(out.metrics or {})
        m.update(compute_rollout_metrics(self.args, samples, time.perf_counter() - t0))
        return samples, m

    def step(self, rollout_id: int) -> dict:
        a = self.args
        t0 = time.perf_counter()
        if self._prefetched is None:
            self._prefetched = self._generate_now(rollout_id)
        samples, metrics = self._prefetched
        self._prefetched = None
        t1 = time.perf_counter()
        fully = getattr(a, "fully_async", False) and hasattr(self.rollout_fn, "pump")
        if fully:
            self.rollout_fn.pump(0.0)
        remote = self.engine is None and self.client is not None
        if remote and rollout_id + 1 < a.num_rollout:
            # the engines are other processes: the next rollout is generated while this one trains, and is drained
            # before the weights change (below)
            self._start_background_generation(rollout_id + 1)
        metrics.update(self.train(rollout_id, samples))
        t2 = time.perf_counter()
        if should_run_periodic_action(rollout_id, a.save_interval, None, a.num_rollout):
            self.actor.save_model(rollout_id)
            self.data_source.save(rollout_id)
        if self._bg is not None:
            self._prefetched = self._collect_background_generation()  # in-flight generation ends before the update
        if (rollout_id + 1) % (a.update_weights_interval or 1) == 0:
            metrics.update(self.update_weights())
        # start the next rollout right away (one-step-async prefetch); with fully-async this mostly drains the buffer
        if self._prefetched is None and rollout_id + 1 < a.num_rollout:
            self._prefetched = self._generate_now(rollout_id + 1)
        t3 = time.perf_counter()
        metrics.update({"perf/train_wait_time": t1 - t0, "perf/train_time": t2 - t1, "perf/step_time": t3 - t0,
                        "perf/wait_time_ratio": (t1 - t0) / max(t3 - t0, 1e-9)})
        if a.eval_interval is not None and should_run_periodic_action(rollout_id, a.eval_interval, None, a.num_rollout):
            metrics.update(self.evaluate(rollout_id))
        if self.tracker is not None:
            self.tracker.log(metrics, step=rollout_id)
        return metrics
