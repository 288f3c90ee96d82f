"""Sampling above the step function: per-request temperature, top-k and seed.

Options and their meaning are the reference's (`temperature`, `top_k`; greedy below 1e-6:
kelpie-engine/kelpie_engine/sdk/engine.py:284-305, kelpie-core/src/request.zig:118-144), plus
a per-request `seed`, which the reference lacks (it keys the draw by the batch,
kelpie-engine/kelpie_engine/sdk/plan.py:96-106). The draw itself is the CUDA kernel in
csrc/kernels/sampling.cu.
"""

from __future__ import annotations

import numpy as np
import torch

from ..kernels import ops


class Sampler:
    def __init__(self, device):
        self.device = torch.device(device)

    def __call__(self, logits: torch.Tensor, temperature, top_k, key0, key1, sample_pos) -> np.ndarray:
        """logits [R, V] float32 on the device; per-row host arrays -> int32 tokens on the host."""
        n = logits.shape[0]
        packed = np.empty((5, n), dtype=np.int32)
        packed[0] = np.asarray(temperature, dtype=np.float32).view(np.int32)
        packed[1] = np.asarray(top_k, dtype=np.int32)
        packed[2] = np.asarray(key0, dtype=np.uint32).view(np.int32)
        packed[3] = np.asarray(key1, dtype=np.uint32).view(np.int32)
        packed[4] = np.asarray(sample_pos, dtype=np.int32)
        dev = torch.from_numpy(packed).to(self.device, non_blocking=True)
        tokens = ops.sample(logits, dev[0].view(torch.float32), dev[1], dev[2], dev[3], dev[4])
        return tokens.cpu().numpy()
