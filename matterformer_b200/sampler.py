"""EDM sampler for the denoiser mirrored in :mod:`matterformer_b200.trunk`.

The stochastic second-order (Heun) sampler of Karras et al. 2022 (Algorithm 2) as the reference applies it to
molecules (src/matterformer/tasks/edm.py:153-233): noise levels ``t_i`` on the rho-schedule, optional churn
(extra noise before each step), an Euler step to ``t_{i+1}`` and a trapezoidal correction, with padded atoms held
at zero and the coordinates re-centred on the real atoms after every update.  A run of ``num_steps`` steps
evaluates the denoiser ``2 * num_steps - 1`` times on tensors of fixed shape, so on CUDA the evaluation is
captured once as a CUDA graph and replayed (``use_cuda_graph``), which removes the launch overhead that dominates
a forward pass over a small batch of small molecules.

Random draws happen in the reference's order (initial atoms, initial coordinates, then per step atoms and
coordinates), so a CPU run with the same global seed reproduces the reference's samples.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .trunk import recenter_coordinates


def build_pad_mask(num_atoms: torch.Tensor, max_atoms: Optional[int] = None) -> torch.Tensor:
    """ref: build_pad_mask, data/qm9.py:94-99.  True marks padding."""
    if num_atoms.ndim != 1:
        raise ValueError(f"num_atoms must have shape (B,), got {tuple(num_atoms.shape)}")
    max_atoms = int(max_atoms or int(num_atoms.max().item()))
    return torch.arange(max_atoms, device=num_atoms.device)[None, :] >= num_atoms[:, None]


def noise_schedule(num_steps: int, sigma_min: float, sigma_max: float, rho: float) -> torch.Tensor:
    """``num_steps`` noise levels from ``sigma_max`` down to ``sigma_min`` plus a final 0 (fp32, on the CPU)."""
    i = torch.arange(num_steps, dtype=torch.float32)
    t = (sigma_max ** (1.0 / rho) + i / max(num_steps - 1, 1) * (sigma_min ** (1.0 / rho) - sigma_max ** (1.0 / rho))) ** rho
    return torch.cat([t, torch.zeros_like(t[:1])])


class GraphedDenoiser:
    """One captured evaluation of ``net`` on fixed-shape buffers, replayed for every noise level.

    Capturing costs a few evaluations; an instance can be handed to several :func:`edm_sample` calls of the same
    batch shape and padding mask (``denoiser=``).
    """

    def __init__(self, net, atoms, coords, pad_mask, lattice, autocast_dtype):
        self.atoms, self.coords = atoms.clone(), coords.clone()
        self.sigma = torch.ones(atoms.shape[0], device=atoms.device)
        self.pad_mask, self.lattice, self.net, self.autocast_dtype = pad_mask, lattice, net, autocast_dtype
        side = torch.cuda.Stream(atoms.device)
        side.wait_stream(torch.cuda.current_stream(atoms.device))
        with torch.cuda.stream(side):  # warm-up outside the capture (lazy initialisation, autotuning)
            for _ in range(2):
                self._eval()
        torch.cuda.current_stream(atoms.device).wait_stream(side)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.out_atoms, self.out_coords = self._eval()

    def _eval(self):
        with torch.autocast("cuda", dtype=self.autocast_dtype, enabled=self.autocast_dtype is not None):
            return self.net(self.atoms, self.coords, self.pad_mask, self.sigma, lattice=self.lattice)

    def __call__(self, atoms, coords, sigma: float):
        self.atoms.copy_(atoms)
        self.coords.copy_(coords)
        self.sigma.fill_(sigma)
        self.graph.replay()
        return self.out_atoms.float(), self.out_coords.float()


@torch.no_grad()
def edm_sample(net, num_atoms: torch.Tensor, *, atom_channels: int = 6, lattice: Optional[torch.Tensor] = None,
               num_steps: int = 100, sigma_min: float = 0.002, sigma_max: float = 10.0, rho: float = 7.0,
               s_churn: float = 30.0, s_min: float = 0.0, s_max: float = float("inf"), s_noise: float = 1.003,
               use_cuda_graph: Optional[bool] = None, autocast_dtype: Optional[torch.dtype] = None,
               denoiser: Optional["GraphedDenoiser"] = None):  # fmt: skip
    """Returns ``(atom_features (B,N,C), coords (B,N,3), pad_mask (B,N))`` like the reference's ``edm_sampler``.

    ``net`` is an :class:`~matterformer_b200.trunk.EDMPreconditioner`.  ``use_cuda_graph`` defaults to "on CUDA for batches of at most 256 molecules";
    ``autocast_dtype`` (e.g. ``torch.bfloat16``) runs the denoiser under autocast.
    """
    device = next(net.parameters()).device
    num_atoms = num_atoms.to(device=device, dtype=torch.long)
    pad_mask = build_pad_mask(num_atoms).to(device)
    batch, max_atoms = pad_mask.shape
    hole = pad_mask[..., None]

    atoms = torch.randn(batch, max_atoms, atom_channels, device=device).masked_fill(hole, 0.0)
    coords = recenter_coordinates(torch.randn(batch, max_atoms, 3, device=device), pad_mask)
    sigma_min = max(float(sigma_min), float(getattr(net, "sigma_min", 0.0)))
    sigma_max = min(float(sigma_max), float(getattr(net, "sigma_max", float("inf"))))
    t_steps = noise_schedule(num_steps, sigma_min, sigma_max, rho)
    atoms = atoms * t_steps[0]
    coords = recenter_coordinates(coords * t_steps[0], pad_mask)

    if use_cuda_graph is None:  # large batches keep the GPU busy without it (measured: no gain at 1024 molecules)
        use_cuda_graph = device.type == "cuda" and batch <= 256
    if denoiser is not None:
        denoise = denoiser
    elif use_cuda_graph:
        denoise = GraphedDenoiser(net, atoms, coords, pad_mask, lattice, autocast_dtype)
    else:
        def denoise(a, c, sigma):
            s = torch.full((batch,), sigma, device=device)
            with torch.autocast(device.type, dtype=autocast_dtype, enabled=autocast_dtype is not None):
                da, dc = net(a, c, pad_mask, s, lattice=lattice)
            return da.float(), dc.float()

    churn = min(s_churn / max(num_steps, 1), math.sqrt(2.0) - 1.0)
    for step in range(num_steps):
        t_cur, t_next = t_steps[step], t_steps[step + 1]
        gamma = churn if s_min <= float(t_cur) <= s_max else 0.0
        t_hat = t_cur + gamma * t_cur
        extra = torch.sqrt(t_hat.square() - t_cur.square()) * s_noise
        atoms_hat = (atoms + extra * torch.randn_like(atoms)).masked_fill(hole, 0.0)
        coords_hat = recenter_coordinates(coords + extra * torch.randn_like(coords), pad_mask)

        den_a, den_c = denoise(atoms_hat, coords_hat, float(t_hat))
        d_a, d_c = (atoms_hat - den_a) / t_hat, (coords_hat - den_c) / t_hat
        atoms = atoms_hat + (t_next - t_hat) * d_a
        coords = recenter_coordinates(coords_hat + (t_next - t_hat) * d_c, pad_mask)
        if step < num_steps - 1:  # trapezoidal correction with the slope at the new point
            den_a, den_c = denoise(atoms, coords, float(t_next))
            t_safe = t_next.clamp_min(1e-8)
            dp_a, dp_c = (atoms - den_a) / t_safe, (coords - den_c) / t_safe
            atoms = atoms_hat + (t_next - t_hat) * 0.5 * (d_a + dp_a)
            coords = recenter_coordinates(coords_hat + (t_next - t_hat) * 0.5 * (d_c + dp_c), pad_mask)
        atoms = atoms.masked_fill(hole, 0.0)
    return atoms, coords, pad_mask
