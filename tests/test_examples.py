"""Every flag that a launch recipe passes exists in the parser (recipes cannot silently rot)."""
import glob
import os
import re

from miles_b200.utils.arguments import build_parser

LAUNCHER_FLAGS = {"--nnodes", "--nproc-per-node", "--master-addr", "--master-port", "--node-rank"}
SERVER_FLAGS = {"--port", "--device", "--max-running-requests", "--page-size", "--context-length", "--host", "--quantization",
                "--mem-fraction-static"}
TOOL_FLAGS = {"--format", "--output"}  # the converter tools of examples/convert_checkpoints.sh (miles_b200/tools)


def test_example_flags_are_known():
    known = set()
    for a in build_parser()._actions:
        known.update(a.option_strings)
    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples")
    files = sorted(glob.glob(os.path.join(root, "*.sh")) + glob.glob(os.path.join(root, "*", "*.sh")))
    assert len(files) >= 8
    for f in files:
        flags = set(re.findall(r"(?<![\w-])(--[a-z][a-z0-9-]+)", open(f).read()))
        unknown = sorted(x for x in flags - known - LAUNCHER_FLAGS - SERVER_FLAGS - TOOL_FLAGS if not x.startswith("--sglang-"))
        assert not unknown, (os.path.basename(f), unknown)


def test_example_config_files_load():
    """The YAML files next to the recipes parse into what their consumers expect."""
    import yaml

    from miles_b200.engine.deployment import Deployment
    from miles_b200.rl.mis import MisOptions
    from types import SimpleNamespace

    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples")
    dep = Deployment.from_yaml(os.path.join(root, "pd_disaggregation.yaml"))
    dep.resolve(SimpleNamespace(hf_checkpoint=None, rollout_num_gpus_per_engine=1))
    kinds = [pl.worker_type for pl in dep.plan(2)]
    assert kinds.count("prefill") == 2 and kinds.count("decode") == 4
    opts = MisOptions.from_args(SimpleNamespace(**yaml.safe_load(open(os.path.join(root, "train_infer_mismatch", "mis.yaml")))))
    assert opts.use_rs and opts.rs_level == "geometric" and opts.tis_batch_normalize
