"""gear/sampler/global_sampler.py: UniformSampler / WeightedSampler / TopKSampler with the
reference's `sync_sample(indices, weights, batch_size)` contract -- every data-parallel rank
gets the same ascending tensor of sampled global indices (:93-152).

What changes underneath:
* the draw runs on the native kernels with variates from a seeded counter-based generator
  (floor(u*n) for the uniform draw, the two-level cumulative table + batched search for the
  weighted one) instead of torch.randint / torch.multinomial;
* every rank generates the same variates, so nobody has to receive the result from rank 0:
  the three point-to-point messages per peer and direction (:22-56) become one all-gather of
  the candidates (and weights) when there is more than one rank;
* the weighted draw is with replacement (external variates cannot drive multinomial's
  without-replacement algorithm).
"""
import numpy as np
import torch
import torch.distributed as dist

from ... import _native as N
from ... import core as _c


def ensure_tensor(v, device="cuda"):
    if isinstance(v, torch.Tensor):
        return v.to(device)
    if isinstance(v, np.ndarray):
        return torch.from_numpy(v).to(device)
    return torch.as_tensor(v).to(device)


class UniformSampler:
    def __init__(self, mpu, seed=42) -> None:
        self._mpu = mpu
        self._seed = int(seed)
        self._calls = 0

    # -- helpers ---------------------------------------------------------------------------
    def _all(self, t: torch.Tensor) -> torch.Tensor:
        """Concatenation of every dp rank's tensor, in rank order (the reference's torch.cat of
        what rank 0 received, :112-116)."""
        world = self._mpu.get_data_parallel_world_size()
        if world == 1:
            return t
        parts = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(parts, t.contiguous(), group=self._mpu.get_data_parallel_group())
        return torch.cat(parts, dim=0)

    def _variates(self, batch_size: int, device) -> torch.Tensor:
        u = torch.empty(batch_size, dtype=torch.float64, device=device)
        _c.fill(u, N.FILL_U01_F64, seed=self._seed, stream_id=self._calls)   # same on every rank
        self._calls += 1
        return u

    # -- the reference's entry points ------------------------------------------------------
    def sync_sample(self, indices, weights, batch_size):
        device = self._mpu.device
        concat_indices = self._all(ensure_tensor(indices, device).to(torch.int64))
        self._cache = self._draw(concat_indices, weights, batch_size, device)
        return torch.sort(concat_indices[self._cache]).values

    def _draw(self, concat_indices, weights, batch_size, device):
        return _c.sample_uniform(concat_indices.numel(), self._variates(batch_size, device))


class WeightedSampler(UniformSampler):
    def __init__(self, mpu, seed=42) -> None:
        super().__init__(mpu, seed)
        self._sampler = None

    def _draw(self, concat_indices, weights, batch_size, device):
        w = self._all(ensure_tensor(weights, device).to(torch.float32).contiguous())
        if w.numel() != concat_indices.numel():
            raise RuntimeError("WeightedSampler: one weight per candidate index is required")
        if self._sampler is None or self._sampler.n != w.numel():
            self._sampler = _c.PrioritySampler(w.numel())
        self._sampler.scan(w)
        return self._sampler.search(self._variates(batch_size, device), scale=True)


class TopKSampler(UniformSampler):
    def _draw(self, concat_indices, weights, batch_size, device):
        w = self._all(ensure_tensor(weights, device).to(torch.float32))
        return torch.topk(input=w, k=batch_size, dim=0, largest=True).indices
