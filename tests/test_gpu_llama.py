"""The Llama flagship on the GPU kernels against the same model evaluated in fp32 on the CPU."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _models(policy):
    from zenyx_b200.models import LlamaConfig, LlamaModel

    cfg = LlamaConfig.tiny(n_layers=2, d_model=256, n_heads=2, n_kv_heads=1, ffn_dim=512, vocab_size=1024)
    gpu = LlamaModel(cfg, device="cuda", remat=policy, seed=3)
    cpu = LlamaModel(cfg, device="cpu", remat=policy, seed=3, dtype=torch.float32)
    cpu.flat.params.copy_(gpu.flat.params.float().cpu())
    return cfg, gpu, cpu


@pytest.mark.parametrize("policy_name", ["selective", "none", "full", "host_offload", "gate_up_in_first_layer"])
def test_llama_gpu_matches_cpu_fp32(policy_name):
    from zenyx_b200.models import RematPolicy
    from zenyx_b200.ops import _ext

    torch.manual_seed(0)
    policy = (RematPolicy(("x", "attn", "h1", "qkv", "gu"), gu_layers=1) if policy_name == "gate_up_in_first_layer"
              else getattr(RematPolicy, policy_name)())
    cfg, gpu, cpu = _models(policy)
    tokens = torch.randint(0, cfg.vocab_size, (2, 512))
    targets = torch.randint(0, cfg.vocab_size, (2, 512))
    l_cpu = cpu.forward_backward(tokens, targets)
    l_gpu = gpu.forward_backward(tokens.cuda(), targets.cuda())
    if policy_name == "host_offload":   # a second micro-batch reuses the pinned buffers and staging slots
        l_cpu = cpu.forward_backward(tokens, targets)
        l_gpu = gpu.forward_backward(tokens.cuda(), targets.cuda())
        assert len(gpu._off_host) == cfg.n_layers and all(t.is_pinned() for t in gpu._off_host.values())
    _ext.check_status()
    assert abs(l_cpu.item() - l_gpu.item()) < 3e-2
    for name in ["layers.0.wqkv", "layers.1.wd", "layers.0.wgu", "layers.1.wo", "lm_head.weight", "embed.weight",
                 "layers.0.norm1", "final_norm"]:
        a, b = gpu.g(name).float().cpu(), cpu.g(name)
        err = (a - b).norm() / (b.norm() + 1e-12)
        assert err < 6e-2, (name, err.item())


def test_trainer_flagship_loss_decreases():
    from zenyx_b200.models import LlamaConfig
    from zenyx_b200.ops import _ext
    from zenyx_b200.train import Trainer, TrainerConfig

    cfg = LlamaConfig.tiny(n_layers=2, d_model=256, n_heads=2, n_kv_heads=2, ffn_dim=512, vocab_size=512)
    tr = Trainer(cfg, TrainerConfig(lr=2e-3, seq_len=256, global_batch=4, max_grad_norm=1.0))
    tok = torch.randint(0, 512, (4, 256))
    losses = [tr.train_step(tok, tok) for _ in range(6)]
    _ext.check_status()
    assert losses[-1] < losses[0] - 0.2, losses
    assert _ext.launch_count > 0
    tr.close()
