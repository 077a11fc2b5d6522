"""Per-coordinate key compressor with the reference toolkit's interface.

Drop-in for ``PerCoordCompressor`` / ``batched_roundtrip`` / ``stack_per_head`` /
``build_method_compressor`` of experiments/stage1/toolkit/per_coord_quantization.py, with the
work done by the CUDA kernels behind ``libjointqk_b200.so``:

* ``roundtrip(states)`` = ``decompress(compress(states))`` and matches the reference
  ``roundtrip`` (:123-165) to fp32 summation-order noise;
* ``compress`` returns real packed pages (``PackedKeys``), which the reference never had;
* ``fit`` wraps the host-side recipe basis -> diagonal products -> water-fill -> integer
  bits -> codebooks (:307-316, :360-389) with the cap on bits per coordinate as a parameter.

There is no CPU implementation here: tensors that live on the host are moved to the GPU for
the call and the result is moved back; without a CUDA device the calls raise.
"""

from __future__ import annotations

import torch

from . import paged
from .allocation import allocate_bits_for_budget, round_bits_to_integer, water_fill
from .basis import eigvec_desc, jointqk_basis
from .codebooks import unit_gaussian_centroids
from .tables import HeadTables


def _cuda_device(pref: torch.device | None = None) -> torch.device:
    if pref is not None and pref.type == "cuda":
        return pref
    if not torch.cuda.is_available():
        raise RuntimeError("jointqk_b200 needs a CUDA device: the key path has no CPU implementation")
    return torch.device("cuda", torch.cuda.current_device())


class PerCoordCompressor:
    """Per-coordinate scalar quantiser with optional pre/post linear maps.

    Args (as the reference constructor, per_coord_quantization.py:69-94):
        bits_per_coord: (d,) integer tensor; 0 bits collapses the coordinate to zero.
        std_per_coord:  (d,) float tensor, standard deviation in the transformed basis.
        forward_map:    (d, d) or None; ``transformed = states @ forward_map``.
        inverse_map:    (d, d) or None; ``recon = quantised @ inverse_map``; defaults to
                        ``forward_map.T`` (orthogonal case).
    """

    def __init__(self, bits_per_coord: torch.Tensor, std_per_coord: torch.Tensor,
                 forward_map: torch.Tensor | None = None, inverse_map: torch.Tensor | None = None) -> None:
        if bits_per_coord.dim() != 1 or std_per_coord.dim() != 1:
            raise ValueError("bits_per_coord and std_per_coord must be 1D")
        if bits_per_coord.shape != std_per_coord.shape:
            raise ValueError("shape mismatch between bits_per_coord and std_per_coord")
        self.d = int(bits_per_coord.shape[0])
        if forward_map is not None and forward_map.shape != (self.d, self.d):
            raise ValueError(f"forward_map must be (d, d) = ({self.d}, {self.d}), got {tuple(forward_map.shape)}")
        self.bits_int = bits_per_coord.round().clamp_min(0).to(torch.long)
        self.stds = std_per_coord.float()
        self.forward_map = forward_map.float() if forward_map is not None else None
        if forward_map is not None and inverse_map is None:
            inverse_map = forward_map.transpose(-1, -2)
        self.inverse_map = inverse_map.float() if inverse_map is not None else None
        self._build_codebooks()
        self._tables: HeadTables | None = None
        self._dense = None
        self._packable: bool | None = None
        self.allocation = "given"          # how bits_per_coord was obtained (set by fit / the builders)

    @property
    def packable(self) -> bool:
        """True when the packed GPU format can store the codes: at most 8 bits per coordinate, at
        most 32 coordinates above 4 bits (those take a byte each) and at most 512 bits per record.
        The reference's default cap of 8 (per_coord_quantization.py:367) fits up to budgets of about
        3 bits per coordinate; beyond the format, ``roundtrip`` and ``codes`` run unpacked
        (``dense.DenseTables``) and there is no cache to attend over."""
        if self._packable is None:
            from .layout import plan_key_layout

            self._packable = True
            if self.bits_int.numel():
                try:
                    plan_key_layout(self.bits_int.cpu().numpy())
                except ValueError:
                    self._packable = False
        return self._packable

    @property
    def decodable(self) -> bool:
        """True when the decode and score kernels can read the codes through their lookup tables: the
        tables of a head (16 entries per group of up to 4 bits, 2^width entries per coordinate of 5..8
        bits) fit the kernels' table memory.  The reference's default allocation (cap 8) fits on the
        configs of its evaluation; an object that does not fit still compresses, unpacks and
        reconstructs on the GPU and is scored from its reconstruction."""
        if not self.packable:
            return False
        from .layout import plan_key_layout

        return plan_key_layout(self.bits_int.cpu().numpy()).decodable if self.bits_int.numel() else True

    def _build_codebooks(self) -> None:
        """(d, K_max) table: row j = unit Gaussian centroids(b_j) * float(std_j), +inf padded;
        a 0-bit row is [0.0] (reference :96-110)."""
        bits = [int(b) for b in self.bits_int.tolist()]
        k_max = max([1] + [2 ** b for b in bits])
        cb = torch.full((self.d, k_max), float("inf"))
        lens = torch.zeros(self.d, dtype=torch.long)
        stds = self.stds.detach().cpu()
        for j, b in enumerate(bits):
            if b == 0:
                cb[j, 0] = 0.0
                lens[j] = 1
            else:
                c = unit_gaussian_centroids(b) * float(stds[j])
                cb[j, : c.numel()] = c
                lens[j] = c.numel()
        self.codebooks_padded = cb
        self.codebook_lengths = lens

    def to(self, device: str | torch.device) -> "PerCoordCompressor":
        self.bits_int = self.bits_int.to(device)
        self.stds = self.stds.to(device)
        self.codebooks_padded = self.codebooks_padded.to(device)
        self.codebook_lengths = self.codebook_lengths.to(device)
        if self.forward_map is not None:
            self.forward_map = self.forward_map.to(device)
        if self.inverse_map is not None:
            self.inverse_map = self.inverse_map.to(device)
        return self

    # -- device tables -------------------------------------------------------------------
    def head_tables(self, device: torch.device | None = None) -> HeadTables:
        dev = _cuda_device(device)
        if not self.packable:
            raise ValueError(
                f"this compressor gives a coordinate {int(self.bits_int.max())} bits and "
                f"{int((self.bits_int > 4).sum())} coordinates more than 4; the packed GPU format stores 0..8 bits per "
                "coordinate with at most 32 coordinates above 4 bits and 512 bits per key.  roundtrip() and codes() "
                "work without a record up to 8 bits per coordinate; for a packed cache fit it with a lower cap "
                "(PerCoordCompressor.fit(..., max_bits=...) or build_method_compressor(..., max_bits=...))")
        if self._tables is None or self._tables.device != dev:
            self._tables = HeadTables.from_compressors([self], device=dev)
        return self._tables

    # -- fit -----------------------------------------------------------------------------
    @classmethod
    def fit(cls, sigma_q: torch.Tensor | None, sigma_k: torch.Tensor, b_avg: float, max_bits: int = 4,
            basis: str = "r_sym", eps: float = 1e-4, allocation: str = "capped_tail") -> "PerCoordCompressor":
        """Fit one head from second moments.

        ``basis="r_sym"``: joint Q-K eigenbasis, water-fill on ``diag(R^T Sq R) * diag(R^T Sk R)``
        (per_coord_quantization.py:307-316,362).  ``basis="sigma_k"``: eigenbasis of Sigma_K and
        water-fill on its variances alone (no query statistics), as the reference's V-side
        compressor does.  ``max_bits`` is the cap on bits per coordinate (the reference hard-codes 8,
        :367; the packed format here stores at most 4).  There are two legitimate ways to honour a
        cap and they give different integer allocations; ``allocation`` picks one and the fitted
        object records it in ``.allocation``:

        * ``"capped_tail"`` (default): the production tail -- uncapped water-fill, largest-remainder
          rounding, clamp at the cap, hand the removed bits to the least-served coordinates
          (:360-379 with the cap as a parameter);
        * ``"water_fill_max"``: the cap goes into the continuous water-fill itself
          (``water_fill(max_bits=cap)``, metric_transform.py:156-213), then the same rounding.

        With outlier channels a cap of 4 costs retrieval quality whichever way it is applied (the
        outliers want 6-8 bits); ``max_bits=8`` gives the reference's allocation, which the host
        objects accept but the packed GPU format cannot store."""
        sk = sigma_k.detach().float().cpu()
        d = sk.shape[-1]
        if basis == "r_sym":
            if sigma_q is None:
                raise ValueError("basis='r_sym' requires sigma_q")
            sq = sigma_q.detach().float().cpu()
            R = jointqk_basis(sq, sk, eps)
            weights = (R.transpose(-1, -2) @ sq @ R).diagonal(dim1=-2, dim2=-1).clamp_min(1e-30)
        elif basis == "sigma_k":
            R = eigvec_desc(sk, eps)
            weights = torch.ones(d)
        else:
            raise ValueError(f"Unknown basis '{basis}'")
        var_k = (R.transpose(-1, -2) @ sk @ R).diagonal(dim1=-2, dim2=-1).clamp_min(1e-30)
        scores = (weights * var_k).unsqueeze(0)
        if allocation == "capped_tail":
            bits = allocate_bits_for_budget(scores, float(b_avg) * d, int(max_bits)).squeeze(0)
        elif allocation == "water_fill_max":
            cont = water_fill(scores.clamp_min(1e-30), total_bits=float(b_avg) * d, max_bits=float(max_bits))
            bits = round_bits_to_integer(cont, total_bits=int(float(b_avg) * d)).squeeze(0).clamp_max(int(max_bits))
        else:
            raise ValueError(f"Unknown allocation '{allocation}'")
        comp = cls(bits, torch.sqrt(var_k.float()), forward_map=R.float(), inverse_map=R.transpose(-1, -2).float())
        comp.allocation = f"{allocation}(max_bits={int(max_bits)})"
        return comp

    # -- compress / decompress / roundtrip ------------------------------------------------
    @torch.no_grad()
    def compress(self, states: torch.Tensor) -> paged.PackedKeys:
        """states (..., d) of any float dtype -> packed pages (one sequence of all rows)."""
        if states.shape[-1] != self.d:
            raise ValueError(f"states last-dim {states.shape[-1]} != compressor.d {self.d}")
        dev = _cuda_device(states.device)
        tables = self.head_tables(dev)
        flat = states.reshape(-1, self.d)
        if flat.dtype not in (torch.float32, torch.bfloat16, torch.float16):
            flat = flat.float()
        flat = flat.to(dev).contiguous()
        packed = paged.compress(tables, flat.view(1, 1, flat.shape[0], self.d))
        packed.leading_shape = tuple(states.shape[:-1])
        return packed

    @torch.no_grad()
    def decompress(self, packed: paged.PackedKeys) -> torch.Tensor:
        out = paged.decompress(packed)            # (1, 1, N, d)
        return out.reshape(tuple(packed.leading_shape) + (self.d,))

    def _unpacked(self, device: torch.device):
        """Tables of the record-free path, for an allocation the packed format does not hold (None
        when it does).  Above 8 bits per coordinate nothing on the GPU applies: ``head_tables`` raises."""
        if self.packable:
            return None
        if int(self.bits_int.max()) > 8:
            self.head_tables(device)          # raises with the explanation
        from .dense import DenseTables

        if self._dense is None or self._dense.device != device:
            eye = torch.eye(self.d)
            fwd = self.forward_map if self.forward_map is not None else eye
            inv = self.inverse_map if self.inverse_map is not None else eye
            self._dense = DenseTables(fwd.unsqueeze(0), inv.unsqueeze(0), self.codebooks_padded.unsqueeze(0), device)
        return self._dense

    @torch.no_grad()
    def codes(self, states: torch.Tensor) -> torch.Tensor:
        """uint8 codes (..., d) the quantiser assigns (the reference's implicit argmin)."""
        dense = self._unpacked(_cuda_device(states.device))
        if dense is not None:
            _, codes = dense.roundtrip(states.reshape(1, -1, self.d), want_out=False, want_codes=True)
            return codes.reshape(tuple(states.shape[:-1]) + (self.d,)).to(states.device)
        packed = self.compress(states)
        return paged.unpack_codes(packed).reshape(tuple(states.shape[:-1]) + (self.d,)).to(states.device)

    @torch.no_grad()
    def roundtrip(self, states: torch.Tensor) -> torch.Tensor:
        """states (..., d) -> fp32 reconstruction of the same shape on ``states.device``."""
        if states.shape[-1] != self.d:
            raise ValueError(f"states last-dim {states.shape[-1]} != compressor.d {self.d}")
        dense = self._unpacked(_cuda_device(states.device))
        if dense is not None:
            out, _ = dense.roundtrip(states.reshape(1, -1, self.d))
            return out.reshape(tuple(states.shape)).to(states.device)
        return self.decompress(self.compress(states)).to(states.device)


def stack_per_head(comps: list[PerCoordCompressor]) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """(forward_maps, inverse_maps, codebooks) of H compressors; codebooks +inf padded to the
    widest (reference :219-233)."""
    d = comps[0].d
    k_max = max(int(c.codebooks_padded.shape[1]) for c in comps)
    cb = torch.full((len(comps), d, k_max), float("inf"))
    for h, c in enumerate(comps):
        cb[h, :, : c.codebooks_padded.shape[1]] = c.codebooks_padded
    fwd = torch.stack([c.forward_map for c in comps], dim=0)
    inv = torch.stack([c.inverse_map for c in comps], dim=0)
    return fwd, inv, cb


_BATCHED_TABLES: dict[tuple, object] = {}


def _codebooks_packable(codebooks: torch.Tensor) -> bool:
    """Whether every head's allocation, read off its (d, K) +inf padded codebook, fits the packed record."""
    from .layout import plan_key_layout

    lengths = torch.isfinite(codebooks.detach().float().cpu()).sum(-1)
    if int(lengths.max()) > 256 or int(lengths.min()) < 1:
        return True                       # not a case for the record-free path: HeadTables raises with the reason
    bits = torch.log2(lengths.float()).round().long()
    try:
        for h in range(bits.shape[0]):
            plan_key_layout(bits[h].numpy())
    except ValueError:
        return False
    return True


def _tables_for(forward_maps, inverse_maps, codebooks, device):
    key = (forward_maps.data_ptr(), inverse_maps.data_ptr(), codebooks.data_ptr(),
           forward_maps._version, inverse_maps._version, codebooks._version, str(device))
    hit = _BATCHED_TABLES.get(key)
    if hit is None:
        if len(_BATCHED_TABLES) > 256:
            _BATCHED_TABLES.clear()
        if _codebooks_packable(codebooks):
            hit = HeadTables(forward_maps, inverse_maps, codebooks, device=device)
        else:
            from .dense import DenseTables

            hit = DenseTables(forward_maps, inverse_maps, codebooks, device)
        _BATCHED_TABLES[key] = hit
    return hit


@torch.no_grad()
def batched_roundtrip(states: torch.Tensor, forward_maps: torch.Tensor, inverse_maps: torch.Tensor,
                      codebooks: torch.Tensor) -> torch.Tensor:
    """All heads of one layer: states (B, H, S, d) -> reconstruction in ``states.dtype``
    (reference :176-216).  One compress launch and one decompress launch for the layer."""
    B, H, S, d = states.shape
    dev = _cuda_device(states.device)
    x = states.to(dev)
    if x.dtype not in (torch.float32, torch.bfloat16, torch.float16):
        x = x.float()
    tables = _tables_for(forward_maps, inverse_maps, codebooks, dev)
    if not isinstance(tables, HeadTables):        # an allocation beyond the packed format: no record in between
        out = torch.stack([tables.roundtrip(x[b])[0] for b in range(B)]) if B else x.float()
        return out.to(states.dtype).to(states.device)
    packed = paged.compress(tables, x)
    return paged.decompress(packed).to(states.dtype).to(states.device)


def build_method_compressor(method: str, sigma_q_for_head: torch.Tensor, sigma_k_for_head: torch.Tensor,
                            cca=None, mq_eigvals=None, mq_eigvecs=None, b_avg: float = 2.0, r: int | None = None,
                            seed: int = 0, head_dim: int = 128, V_h=None, R_sym: torch.Tensor | None = None,
                            max_bits: int = 8) -> PerCoordCompressor | None:
    """Reference signature (:261-274) for the method on this path, ``r_sym_waterfill``.

    ``max_bits`` defaults to the reference's hard-coded 8 (:367), so the object built here has the
    reference's bits, standard deviations and codebooks.  The packed GPU format stores up to 8 bits
    per coordinate (a byte each above 4 bits, at most 32 such coordinates per head) and the decode
    kernels read them (``.packable``, ``.decodable``); ``max_bits=4`` is a different allocation
    with a quality cost where outlier channels want more than 4 bits, so it is never substituted
    silently.  Other method ids belong
    to ablations outside this build and raise ``ValueError`` like an unknown method does in the
    reference."""
    if method == "v3":
        return None
    if method != "r_sym_waterfill":
        raise ValueError(f"Unknown method '{method}'")
    if R_sym is None:
        raise ValueError("r_sym_* methods require R_sym")
    R = R_sym.float()
    var_k = (R.transpose(-1, -2) @ sigma_k_for_head.float() @ R).diagonal(dim1=-2, dim2=-1).clamp_min(1e-30)
    weights = (R.transpose(-1, -2) @ sigma_q_for_head.float() @ R).diagonal(dim1=-2, dim2=-1).clamp_min(1e-30)
    bits = allocate_bits_for_budget((weights * var_k).unsqueeze(0), float(b_avg) * head_dim, int(max_bits)).squeeze(0)
    comp = PerCoordCompressor(bits, torch.sqrt(var_k.float()), forward_map=R, inverse_map=R.transpose(-1, -2))
    comp.allocation = f"capped_tail(max_bits={int(max_bits)})"
    return comp
