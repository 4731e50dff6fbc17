"""CPU stand-in for a train engine, used by the scheduler / controller tests."""
import torch


class FakeTrainEngine:
    def __init__(self, scale: float = 1.0):
        self.scale = scale
        self.calls = 0
        self.version = 0
        self.rank = 0

    def train_batch(self, data, *args, **kwargs):
        self.calls += 1
        s = float(sum(v.sum() for v in data.values() if torch.is_tensor(v)))
        return {"sum": s * self.scale, "calls": self.calls, "n": float(sum(v.shape[0] for v in data.values() if torch.is_tensor(v)))}

    def forward_batch(self, data, *args, **kwargs):
        return data["input_ids"].float() * self.scale

    def make_batch(self, n):
        return {"ids": torch.arange(n)}

    def consume(self, batch):
        return int(batch["ids"].sum())

    def set_version(self, v):
        self.version = v

    def get_version(self):
        return self.version

    def explode(self):
        raise RuntimeError("engine failure")
