"""Example 01: any ``nn.Module`` through the Trainer, on whatever device is there.

    python examples/01_quickstart_any_module.py

The counterpart of the reference's beginner example (examples/01_beginner_cpu_training.py): a small
token model, synthetic data, a couple of epochs. The difference is that the loop is the framework's
``Trainer.train_step(batch, target, criterion)`` (the reference's public API, zenyx/train/trainer.py:36-57)
rather than hand-written ``backward()`` / ``step()`` calls.
"""
import json
import sys
from pathlib import Path

import torch
import torch.nn as nn

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
from zenyx_b200.train import Trainer, TrainerConfig  # noqa: E402


class TokenLoss(nn.Module):
    def forward(self, logits, target):
        return nn.functional.cross_entropy(logits.reshape(-1, logits.shape[-1]), target.reshape(-1))


def main(epochs: int = 2, out: str = "example01_metrics.json"):
    torch.manual_seed(0)
    vocab, hidden, seq, batch = 1000, 64, 32, 4
    model = nn.Sequential(nn.Embedding(vocab, hidden), nn.Linear(hidden, hidden), nn.ReLU(), nn.Linear(hidden, vocab))
    trainer = Trainer(model, TrainerConfig(lr=1e-3, max_grad_norm=1.0))
    inputs = torch.randint(0, vocab, (100, seq))
    targets = (inputs + 1) % vocab                      # a learnable rule: next token id
    crit, history = TokenLoss(), []
    for epoch in range(epochs):
        losses = [trainer.train_step(inputs[i:i + batch], targets[i:i + batch], crit) for i in range(0, 100, batch)]
        history.append(sum(losses) / len(losses))
        print(f"epoch {epoch + 1}: mean loss {history[-1]:.4f}")
    Path(out).write_text(json.dumps({"epoch_loss": history}))
    trainer.close()
    return history


if __name__ == "__main__":
    main()
