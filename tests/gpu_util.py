"""Helpers shared by the GPU parity tests."""
import torch

ULP = 2.0 ** -7      # one bf16 unit in the last place, relative to the value's binade


def rel_fro(got: torch.Tensor, want: torch.Tensor) -> float:
    got, want = got.double().cpu(), want.double().cpu()
    return ((got - want).norm() / want.norm().clamp_min(1e-30)).item()


def within_ulps(got: torch.Tensor, want: torch.Tensor, ulps: float = 1.0, floor: float = 1e-6):
    """Every element within `ulps` bf16 ulps of `want` (absolute floor for values near zero)."""
    got, want = got.float().cpu(), want.float().cpu()
    tol = ulps * ULP * want.abs() + floor
    return bool(((got - want).abs() <= tol).all())


def mismatch_fraction(got: torch.Tensor, want: torch.Tensor) -> float:
    return (got.cpu().view(torch.int16) != want.cpu().view(torch.int16)).float().mean().item()


def seeded(shape, seed, scale=1.0, device="cuda"):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(torch.bfloat16).to(device)
