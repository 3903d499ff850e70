"""Newton-Schulz drivers with the reference's signatures (ancora/kernels/muon_ns.py).

``newton_schulz_resident`` / ``newton_schulz_resident_e`` keep the reference's argument
lists (muon_ns.py:245,430): packed bf16 operand ``gX`` overwritten with the result,
caller-owned scratch ``gA, gA2, gB, gBX`` and ``grecip``.  The chain itself runs in the
library's tcgen05 kernels; ``gA2`` is accepted and left untouched (the fused chain never
materialises A@A, as in the reference's ``fused=True`` path).  ``fused=False``, which in the
reference selects the chain of separate matmul / axpy launches (muon_ns.py:277-283), here
selects one launch per phase instead of the single persistent launch; the arithmetic and
the resulting bits are the same.
"""
from .kernels import ns_batched

NTM, NTN, NTK = 128, 128, 64
A_COEF, B_COEF, C_COEF = 3.4445, -4.7750, 2.0315

# Polar-Express per-iteration coefficients (muon_ns.py:30-34)
PE_SCHEDULE = [(4.0848, -6.8946, 2.9270),
               (3.9505, -6.3029, 2.6377),
               (3.7418, -5.5913, 2.3037),
               (2.8769, -3.1427, 1.2046),
               (2.8366, -3.0525, 1.2012)]

_KELLER = object()
_DEFAULT_SCHEDULE = None


def _coef_at(schedule, k):
    """(a,b,c) of iteration k: Keller if schedule is None, else schedule[k] with the last
    triple repeated past the end (muon_ns.py:37-42)."""
    if schedule is None:
        return A_COEF, B_COEF, C_COEF
    return schedule[k] if k < len(schedule) else schedule[-1]


def set_polar_express(on: bool):
    """Process-wide default schedule for callers that pass none; returns the previous
    setting (muon_ns.py:55-61)."""
    global _DEFAULT_SCHEDULE
    prev = _DEFAULT_SCHEDULE
    _DEFAULT_SCHEDULE = PE_SCHEDULE if on else None
    return prev


def _resolve(schedule):
    return _DEFAULT_SCHEDULE if schedule is _KELLER else schedule


def coeff_list(schedule, steps):
    return [tuple(_coef_at(schedule, k)) for k in range(steps)]


def _check(M, N):
    assert M <= N, f"Newton-Schulz needs M <= N, got ({M},{N}); transpose tall weights first"
    assert M % NTM == 0 and N % NTN == 0, f"NS shape ({M},{N}) tile-misaligned"


def newton_schulz_resident(gX, gA, gA2, gB, gBX, grecip, M, N, si, steps=5, eps=1e-7,
                           schedule=_KELLER, fused=True):
    _check(M, N)
    ns_batched(gX, gA, gB, gBX, grecip, 1, M, N, steps, coeff_list(_resolve(schedule), steps), eps, si,
               single_launch=bool(fused))


def newton_schulz_resident_e(gX, gA, gA2, gB, gBX, grecip, E, M, N, si, steps=5, eps=1e-7,
                             schedule=_KELLER, fused=True):
    _check(M, N)
    ns_batched(gX, gA, gB, gBX, grecip, E, M, N, steps, coeff_list(_resolve(schedule), steps), eps, si,
               single_launch=bool(fused))
