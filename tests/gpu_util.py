"""Helpers shared by the GPU parity tests."""

import numpy as np
import torch

from oracle import reference_port as orc


def code_mismatch(codes_gpu: torch.Tensor, codes_ref: torch.Tensor) -> tuple[int, float]:
    bad = int((codes_gpu.cpu().to(torch.int16) != codes_ref.cpu().to(torch.int16)).sum())
    return bad, bad / max(1, codes_ref.numel())


def oracle_codes_and_recon(comp, keys: torch.Tensor):
    """Reference-algorithm codes and reconstruction of one head on the CPU."""
    out, codes = orc.roundtrip(keys.cpu(), comp.codebooks_padded.cpu(), comp.forward_map.cpu(), comp.inverse_map.cpu())
    return codes, out


def recon_from_codes(comp, codes: torch.Tensor) -> torch.Tensor:
    """k_hat for given codes (N, d) with the reference's gather + inverse map."""
    xh = orc.dequantise(codes.long().cpu(), comp.codebooks_padded.cpu())
    return xh @ comp.inverse_map.cpu()


def score_rel_error(s: torch.Tensor, ref: torch.Tensor) -> float:
    """max_i |s_i - ref_i| / max(|ref_i|, rms_row(ref)) -- the score tolerance metric."""
    rms = ref.pow(2).mean(-1, keepdim=True).sqrt()
    return float(((s - ref).abs() / torch.maximum(ref.abs(), rms)).max())
