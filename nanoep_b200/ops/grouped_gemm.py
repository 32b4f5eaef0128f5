"""Grouped GEMM over expert-major rows (tcgen05 / TMEM kernel, csrc/grouped_gemm_sm100.cu).

``rows`` come from a dispatch with ``do_expand=True, alignment=128, zero_padding=True``: every
128-row block belongs to one expert, padding rows are zero.  The reference library stops at
dispatch/combine; these ops are the expert compute that sits between them on the same GPU.
"""

from __future__ import annotations

import torch

PLAIN, SWIGLU = 0, 1
_status: dict[int, torch.Tensor] = {}


def _ext():
    from ..utils.build import load_extension

    return load_extension()


def status_tensor(device) -> torch.Tensor:
    index = torch.device(device).index
    if index is None:
        index = torch.cuda.current_device()
    if index not in _status:
        _status[index] = torch.zeros(4, dtype=torch.int32, device=torch.device("cuda", index))
    return _status[index]


def check_status(device=None):
    """Raise if a GEMM kernel on ``device`` gave up on a bounded wait (synchronises)."""
    st = status_tensor(device if device is not None else torch.cuda.current_device())
    code, cta = (int(v) for v in st[:2].tolist())
    if code != 0:
        st.zero_()
        reasons = {101: "an operand pipeline wait timed out", 102: "the wait for a row block's ready counter timed out",
                   103: "expert_offsets are not multiples of 128 from 0 to the row count", 104: "handle metadata names an impossible rank, token or row"}
        raise RuntimeError(f"nanoep_b200 grouped GEMM status {code} ({reasons.get(code, 'unknown')}), detail {cta}")


def grouped_gemm(a, w, expert_offsets, *, swiglu: bool = False, out=None, tile_ready=None, tile_expected=None, max_ctas: int = 0,
                 timeout_s: float = 5.0, row_scale=None, stages: int = 4, pair: bool = False) -> torch.Tensor:
    """``out[r] = a[r] @ w[e(r)].T`` (bf16 in, fp32 accumulate, bf16 out).

    a: ``[rows, K]`` bf16, rows % 128 == 0;  w: ``[E, N, K]`` bf16 (``[E, 2*I, K]`` gate rows then up
    rows when ``swiglu``);  expert_offsets: int64 ``[E+1]`` row offsets (multiples of 128).
    With ``swiglu`` the result is ``silu(a @ w_gate.T) * (a @ w_up.T)`` of shape ``[rows, I]``.
    ``row_scale`` (fp32 ``[rows]``, plain mode) multiplies each output row in FP32 before the bf16 round.
    ``stages=3`` shrinks the operand pipeline so that a transfer kernel can share the SMs.
    ``pair=True`` runs the CTA-pair kernel (tcgen05 ``cta_group::2``: two SMs share every weight tile).
    """
    n_out = w.shape[1] // 2 if swiglu else w.shape[1]
    if out is None:
        out = torch.empty((a.shape[0], n_out), dtype=torch.bfloat16, device=a.device)
    _ext().grouped_gemm(a, w, expert_offsets, out, status_tensor(a.device), SWIGLU if swiglu else PLAIN, tile_ready, tile_expected,
                        int(max_ctas), float(timeout_s), row_scale, int(stages), bool(pair))
    return out


def grouped_gemm_reference(a, w, expert_offsets, *, swiglu: bool = False) -> torch.Tensor:
    """Plain PyTorch fp32 reference of the same op (for tests)."""
    offsets = expert_offsets.tolist()
    n_out = w.shape[1] // 2 if swiglu else w.shape[1]
    out = torch.zeros((a.shape[0], n_out), dtype=torch.float32, device=a.device)
    for e in range(w.shape[0]):
        lo, hi = offsets[e], offsets[e + 1]
        if hi <= lo:
            continue
        y = a[lo:hi].float() @ w[e].float().t()
        if swiglu:
            inner = w.shape[1] // 2
            y = torch.nn.functional.silu(y[:, :inner]) * y[:, inner:]
        out[lo:hi] = y
    return out
