"""File-backed Adam equals in-memory AdamW; on-policy-distillation advantage correction."""
import math

import torch

from miles_b200.models import ParamStore, get_config
from miles_b200.rl.opd import apply_opd, teacher_logprob_from_topk
from miles_b200.trainer.nvme_optimizer import NvmeStreamedAdam


def test_nvme_adam_matches_torch_adamw(tmp_path):
    cfg = get_config("qwen3-tiny")
    store = ParamStore(cfg, "cpu", torch.float32, seed=2)
    store.allocate_grads(torch.float32)
    ref = {g: t.clone().requires_grad_(True) for g, t in store.flat.items() if t.numel()}
    topt = torch.optim.AdamW(list(ref.values()), lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    opt = NvmeStreamedAdam(store, str(tmp_path), lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1, bucket_elems=50_000, moment_dtype="fp32")
    assert len(opt.buckets) > 3
    gen = torch.Generator().manual_seed(0)
    for _ in range(3):
        for g, t in ref.items():
            gr = torch.randn(t.shape, generator=gen) * 0.01
            store.grad[g].copy_(gr)
            t.grad = gr.clone()
        opt.step()
        topt.step()
    for g, t in ref.items():
        assert torch.allclose(store.flat[g], t.detach(), atol=2e-6, rtol=1e-5), g
    assert opt.bytes_read > 0 and opt.bytes_written > 0
    # a fresh optimizer over the same directory resumes from the files
    again = NvmeStreamedAdam(store, str(tmp_path), lr=1e-2, bucket_elems=50_000)
    m = again._load_bucket(0)[1]
    assert m.abs().sum() > 0


def test_opd_lowers_advantage_where_student_is_overconfident():
    adv = torch.zeros(4)
    s = torch.tensor([-0.1, -2.0, -1.0, -0.5])
    t = torch.tensor([-1.1, -2.0, -0.5, -0.5])
    out, kl = apply_opd(adv, s, t, opd_kl_coef=0.5, loss_mask=torch.tensor([1, 1, 1, 0]))
    assert torch.allclose(out, torch.tensor([-0.5, 0.0, 0.25, 0.0]))
    assert abs(float(kl) - (1.0 + 0.0 - 0.5) / 3) < 1e-6
    lp = teacher_logprob_from_topk(7, [1, 2], [math.log(0.5), math.log(0.3)], vocab_size=12)
    assert abs(lp - math.log(0.2 / 10)) < 1e-9
    assert teacher_logprob_from_topk(2, [1, 2], [math.log(0.5), math.log(0.3)], 12) == math.log(0.3)
