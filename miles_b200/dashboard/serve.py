"""Serve the dashboard of a run (live or finished):

    python -m miles_b200.dashboard.serve --dump-details /runs/exp1 [--hf-checkpoint /models/Qwen3-4B] [--port 8265]

``--dump-details`` is the run's ``--dump-details`` directory: the event store lives under ``dashboard/``, the rollout
dumps the inspector reads under ``rollout_data/``. With ``--hf-checkpoint`` tokens are shown with their text.
Reference counterpart: miles/dashboard/serve.py.
"""
import argparse
import os


def build(dump_details: str, hf_checkpoint: str = None):
    from . import EventStore, build_dashboard_app
    from .dump_reader import DumpReader

    tokenizer = None
    if hf_checkpoint:
        from ..utils.processing_utils import load_tokenizer

        tokenizer = load_tokenizer(hf_checkpoint)
    store = EventStore(os.path.join(dump_details, "dashboard"))
    return build_dashboard_app(store, DumpReader(os.path.join(dump_details, "rollout_data"), tokenizer))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--dump-details", required=True)
    ap.add_argument("--hf-checkpoint", default=None)
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8265)
    a = ap.parse_args()
    import uvicorn

    uvicorn.run(build(a.dump_details, a.hf_checkpoint), host=a.host, port=a.port, log_level="warning")


if __name__ == "__main__":
    main()
