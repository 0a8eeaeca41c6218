"""CPU oracle for the contrastive-loss path.  TEST INFRASTRUCTURE ONLY.

Nothing in the shipped package imports this module: it is the checker used by
``tests/``, by ``__graft_entry__.smoke()`` and by the CPU-baseline leg of
``bench.py``.  The product path is the CUDA library and fails without it.

Two independent statements of the same mathematics live here:

* ``clip_dense`` / ``lit_dense`` - the dense PyTorch formulation
  ``0.5 * (CE(x y^T / T, diag) + CE(y x^T / T, diag))`` (LiT: one direction)
  differentiated by autograd.  This is the parity reference.
* ``clip_closed_form`` / ``lit_closed_form`` - a numpy restatement of the
  reference's tile algorithm without tiles: fixed-max exponentials, row and
  column sums, loss from the diagonal, and the explicit gradient formulas
  (reference clip_loss.py:56, 59-64, 115-124, 206-211, 235-236, 252-254;
  lit_loss.py:59, 62, 113-120, 199-203, 227).

Pinning: the reference ships no tests or golden vectors.  The closed form is
pinned against the reference's own Triton kernels run on CPU through Triton's
interpreter (``tests/golden/make_golden.py`` writes ``tests/golden/*.npz``),
and against the dense formulation, in ``tests/test_oracle.py``.
"""
from __future__ import annotations

import math

import numpy as np
import torch
import torch.nn.functional as F

LOG2E = 1.4426950408889634


# --------------------------------------------------------------------------- #
# dense formulation (autograd)
# --------------------------------------------------------------------------- #
def _prep(t: torch.Tensor, dtype: torch.dtype, requires_grad: bool) -> torch.Tensor:
    return t.detach().to("cpu").to(dtype).clone().requires_grad_(requires_grad)


def grad_multiplier(batch: int, temperature: float, stable: bool) -> float:
    """Stable variants keep the loss and multiply every gradient by sqrt(B*T).

    Reference clip_loss.py:299 uses sqrt(B/T)/B where the plain variant uses
    1/(B*T) (clip_loss.py:182, 235); the ratio is sqrt(B*T).
    """
    return math.sqrt(batch * temperature) if stable else 1.0


def clip_dense(image, text, temperature=0.07, normalized_inputs=False, stable=False,
               grad_output=1.0, dtype=torch.float64):
    """Dense CLIP loss and gradients w.r.t. the module inputs.

    Mirrors MemoryEfficientCLIPLoss.forward (clip_loss.py:265-273): optional
    F.normalize(dim=1) on both inputs, then the symmetric cross entropy.
    Returns (loss, d_image, d_text) as CPU tensors of ``dtype``.
    """
    x = _prep(image, dtype, True)
    y = _prep(text, dtype, True)
    xn, yn = (x, y) if normalized_inputs else (F.normalize(x, dim=1), F.normalize(y, dim=1))
    logits = xn @ yn.t() / temperature
    labels = torch.arange(x.shape[0])
    loss = 0.5 * (F.cross_entropy(logits, labels) + F.cross_entropy(logits.t(), labels))
    mult = grad_multiplier(x.shape[0], temperature, stable) * grad_output
    gx, gy = torch.autograd.grad(loss, (x, y))
    return loss.detach(), gx * mult, gy * mult


def lit_dense(text, image, temperature=0.07, normalized_inputs=False, stable=False,
              grad_output=1.0, dtype=torch.float64):
    """Dense LiT loss (text -> image direction only), gradient for text only.

    Mirrors MemoryEfficientLiTLoss.forward(text_features, image_features)
    (lit_loss.py:256-263); the image tower is frozen (lit_loss.py:247).
    """
    x = _prep(text, dtype, True)
    y = _prep(image, dtype, False)
    xn, yn = (x, y) if normalized_inputs else (F.normalize(x, dim=1), F.normalize(y, dim=1))
    logits = xn @ yn.t() / temperature
    loss = F.cross_entropy(logits, torch.arange(x.shape[0]))
    mult = grad_multiplier(x.shape[0], temperature, stable) * grad_output
    (gx,) = torch.autograd.grad(loss, (x,))
    return loss.detach(), gx * mult


def temperature_grad_dense(first, second, temperature, kind="clip", normalized_inputs=False, dtype=torch.float64):
    """d loss / d temperature by autograd on the dense formulation (the reference has no such
    gradient: its backward returns None for the temperature, clip_loss.py:256)."""
    x = _prep(first, dtype, False)
    y = _prep(second, dtype, False)
    t = torch.tensor(float(temperature), dtype=dtype, requires_grad=True)
    xn, yn = (x, y) if normalized_inputs else (F.normalize(x, dim=1), F.normalize(y, dim=1))
    logits = xn @ yn.t() / t
    labels = torch.arange(x.shape[0])
    loss = F.cross_entropy(logits, labels)
    if kind == "clip":
        loss = 0.5 * (loss + F.cross_entropy(logits.t(), labels))
    (gt,) = torch.autograd.grad(loss, (t,))
    return float(gt)


def siglip_dense(image, text, logit_scale, logit_bias, normalized_inputs=False, grad_output=1.0, dtype=torch.float64):
    """Dense sigmoid (SigLIP) loss: (1/B) sum_ij softplus(-z_ij (t s_ij + b)), z = 2 I - 1, with
    gradients for both inputs, the scale t and the bias b.  (Not in the reference; the checker of
    the sigmoid-loss extension.)  Returns (loss, d_image, d_text, d_t, d_b)."""
    x = _prep(image, dtype, True)
    y = _prep(text, dtype, True)
    t = torch.tensor(float(logit_scale), dtype=dtype, requires_grad=True)
    b = torch.tensor(float(logit_bias), dtype=dtype, requires_grad=True)
    xn, yn = (x, y) if normalized_inputs else (F.normalize(x, dim=1), F.normalize(y, dim=1))
    a = xn @ yn.t() * t + b
    z = 2.0 * torch.eye(x.shape[0], dtype=dtype) - 1.0
    loss = F.softplus(-z * a).sum() / x.shape[0]
    gx, gy, gt, gb = torch.autograd.grad(loss, (x, y, t, b))
    return loss.detach(), gx * grad_output, gy * grad_output, float(gt) * grad_output, float(gb) * grad_output


# --------------------------------------------------------------------------- #
# closed form: the reference's algorithm without the tiling
# --------------------------------------------------------------------------- #
def sum_exp(xn: np.ndarray, yn: np.ndarray, temperature: float):
    """E = exp2(k*S - k), k = log2(e)/T; row sums r and column sums c.

    Reference clip_loss.py:53-60 (forward tile) with the padding columns left
    out, i.e. what the reference computes when B is a multiple of 128.
    """
    k = LOG2E / temperature
    e = np.exp2(xn @ yn.T * k - k)
    return e, e.sum(axis=1), e.sum(axis=0)


def clip_closed_form(xn, yn, temperature=0.07, stable=False, grad_output=1.0):
    """Loss and gradients w.r.t. *normalised* inputs, numpy float64.

    loss: clip_loss.py:206-211.  G: clip_loss.py:121-124.  Gradient init and
    accumulation: clip_loss.py:235-236, 148-156.  grad_output: :252-254.
    """
    xn = np.asarray(xn, dtype=np.float64)
    yn = np.asarray(yn, dtype=np.float64)
    b = xn.shape[0]
    k = LOG2E / temperature
    e, r, c = sum_exp(xn, yn, temperature)
    sv = np.einsum("bi,bi->b", xn, yn) * k - k
    loss = -(np.log(np.exp2(sv) / r) + np.log(np.exp2(sv) / c)).mean() / 2.0
    scale = math.sqrt(b / temperature) / b if stable else 1.0 / (temperature * b)
    g = (e / r[:, None] + e / c[None, :]) * (scale / 2.0)
    dx = (g @ yn - yn * scale) * grad_output
    dy = (g.T @ xn - xn * scale) * grad_output
    return {"loss": loss, "row_sum": r, "col_sum": c, "dx": dx, "dy": dy}


def lit_closed_form(xn, yn, temperature=0.07, stable=False, grad_output=1.0):
    """LiT: X = text, Y = image; row sums only (lit_loss.py:59-62, 118-120, 199-203, 227)."""
    xn = np.asarray(xn, dtype=np.float64)
    yn = np.asarray(yn, dtype=np.float64)
    b = xn.shape[0]
    k = LOG2E / temperature
    e, r, _ = sum_exp(xn, yn, temperature)
    sv = np.einsum("bi,bi->b", xn, yn) * k - k
    loss = -np.log(np.exp2(sv) / r).mean()
    scale = math.sqrt(b / temperature) / b if stable else 1.0 / (temperature * b)
    g = e / r[:, None] * scale
    dx = (g @ yn - yn * scale) * grad_output
    return {"loss": loss, "row_sum": r, "dx": dx}


def round_tf32(x):
    """fp32 values rounded to the nearest tf32 (10 explicit mantissa bits, ties away from zero: what the PTX
    conversion cvt.rna.tf32.f32 does), returned as fp32 whose 13 low mantissa bits are zero.  This is the operand
    precision of tl.dot on fp32 inputs in the reference (clip_loss.py:53, :113; Triton's default tf32 input
    precision).  Accepts a numpy array or a torch tensor; finite values only."""
    is_torch = isinstance(x, torch.Tensor)
    a = (x.detach().cpu().float().numpy() if is_torch else np.asarray(x, dtype=np.float32)).copy()
    bits = a.view(np.uint32)
    bits += np.uint32(0x1000)              # half a tf32 unit in the last place, added to the magnitude
    bits &= np.uint32(0xFFFFE000)
    return torch.from_numpy(a) if is_torch else a


def normalize_np(x: np.ndarray, eps: float = 1e-12):
    """F.normalize(dim=1): x / max(||x||, eps).  Returns (x_hat, 1/max(||x||, eps))."""
    x = np.asarray(x, dtype=np.float64)
    inv = 1.0 / np.maximum(np.sqrt((x * x).sum(axis=1)), eps)
    return x * inv[:, None], inv


def normalize_jacobian_np(x_hat: np.ndarray, inv_norm: np.ndarray, g_hat: np.ndarray):
    """Backward of F.normalize: dx = (g - x_hat * (x_hat . g)) / ||x||."""
    dot = (x_hat * g_hat).sum(axis=1, keepdims=True)
    return (g_hat - x_hat * dot) * inv_norm[:, None]


# --------------------------------------------------------------------------- #
# streaming form for batches whose B x B matrix does not fit in host memory
# --------------------------------------------------------------------------- #
def clip_streaming(xn: torch.Tensor, yn: torch.Tensor, temperature: float, sample_rows,
                   block: int = 4096, lit: bool = False, dtype=torch.float32):
    """Row-blocked evaluation: exact r, c, loss, and exact gradient rows for
    ``sample_rows`` of d_x and d_y.  O(block * B) memory.  Same formulas as the
    closed form above; used for the ring-distributed configurations.
    """
    xn = xn.to(dtype)
    yn = yn.to(dtype)
    b = xn.shape[0]
    k = LOG2E / temperature
    r = torch.zeros(b, dtype=torch.float64)
    c = torch.zeros(b, dtype=torch.float64)
    for i0 in range(0, b, block):
        e = xn[i0:i0 + block] @ yn.t()              # in place from here on: one [block, B] buffer per trip
        e.mul_(k).sub_(k)
        torch.exp2(e, out=e)
        r[i0:i0 + block] = e.sum(dim=1, dtype=torch.float64)
        c += e.sum(dim=0, dtype=torch.float64)
    sv = ((xn.double() * yn.double()).sum(dim=1) * k - k) * math.log(2.0)
    if lit:
        loss = (torch.log(r) - sv).mean()
    else:
        loss = 0.5 * (torch.log(r) + torch.log(c) - 2 * sv).mean()
    scale = 1.0 / (temperature * b)
    rows = torch.as_tensor(sample_rows, dtype=torch.long)
    # d_x rows: G[rows, :] @ yn - yn[rows] * scale
    e = torch.exp2((xn[rows] @ yn.t()) * k - k).double()
    if lit:
        g = e / r[rows, None] * scale
    else:
        g = (e / r[rows, None] + e / c[None, :]) * (scale / 2)
    dx_rows = g @ yn.double() - yn[rows].double() * scale
    out = {"loss": loss, "row_sum": r, "col_sum": c, "rows": rows, "dx_rows": dx_rows}
    if not lit:
        et = torch.exp2((yn[rows] @ xn.t()) * k - k).double()      # E^T rows: [s, B]
        gt = (et / r[None, :] + et / c[rows, None]) * (scale / 2)
        out["dy_rows"] = gt @ xn.double() - xn[rows].double() * scale
    return out


def clip_blocked_step(xn: torch.Tensor, yn: torch.Tensor, temperature: float, row_block: int = 4096,
                      rows: int | None = None, want_grads: bool = True):
    """The reference's two-kernel algorithm on the host cores, fp32, in row blocks: a forward pass over
    [row_block x B] strips of S = X Y^T for the row and column sums (clip_sum_exp_kernel,
    clip_loss.py:36-64), the loss from the diagonal (clip_loss.py:206-211), then a backward pass that
    RECOMPUTES each strip, forms G = (E/r + E/c) / (2 B T) (clip_loss.py:96-124) and contracts it:
    dX_strip = G Y - Y_strip/(B T), dY += G^T X_strip (clip_loss.py:127-156, 235-236).  Executed FLOPs are
    the 8 B^2 D the throughput metric counts; peak memory is three strips, never B x B.

    rows: work on the first `rows` rows of X only (a bounded SAMPLE of a problem too large to time whole on
    the host: the column sums then cover those rows only and the results are not the loss's, the work per
    row is).  Returns (loss, dX [rows, D], dY [B, D]) - fp32 tensors."""
    xn = xn.float()
    yn = yn.float()
    b, d = yn.shape
    n = b if rows is None else min(rows, xn.shape[0])
    k = LOG2E / temperature
    r = torch.zeros(n, dtype=torch.float32)
    c = torch.zeros(b, dtype=torch.float32)
    yt = yn.t().contiguous()
    for i0 in range(0, n, row_block):
        i1 = min(n, i0 + row_block)
        e = xn[i0:i1] @ yt
        e.mul_(k).sub_(k)
        torch.exp2(e, out=e)
        r[i0:i1] = e.sum(dim=1)
        c += e.sum(dim=0)
    sv = ((xn[:n] * yn[:n]).sum(dim=1) * k - k) * math.log(2.0)
    loss = 0.5 * (torch.log(r) + torch.log(c[:n]) - 2 * sv).mean()
    if not want_grads:
        return loss, None, None
    scale = 1.0 / (temperature * b)
    inv_r = (0.5 * scale) / r
    inv_c = (0.5 * scale) / c
    dx = torch.empty(n, d, dtype=torch.float32)
    dy = torch.zeros(b, d, dtype=torch.float32)
    for i0 in range(0, n, row_block):
        i1 = min(n, i0 + row_block)
        e = xn[i0:i1] @ yt
        e.mul_(k).sub_(k)
        torch.exp2(e, out=e)
        g = e * inv_r[i0:i1, None]
        g.addcmul_(e, inv_c[None, :])
        torch.mm(g, yn, out=dx[i0:i1])
        dx[i0:i1].sub_(yn[i0:i1] * scale)
        dy.addmm_(g.t(), xn[i0:i1])
    dy[:n].sub_(xn[:n] * scale)
    return loss, dx, dy


# --------------------------------------------------------------------------- #
# tolerances (loss 1e-3 relative; gradients 1e-2 max-relative, cosine >= 0.9999)
# --------------------------------------------------------------------------- #
LOSS_RTOL = 1e-3
GRAD_MAX_REL = 1e-2
GRAD_COS_MIN = 0.9999


def loss_rel_err(got, ref) -> float:
    got = float(got)
    ref = float(ref)
    return abs(got - ref) / max(abs(ref), 1e-30)


def grad_errors(got, ref):
    """(max|got-ref| / max|ref|, cosine similarity) over the whole tensor."""
    g = torch.as_tensor(np.asarray(got.detach().cpu().double()) if isinstance(got, torch.Tensor) else got,
                        dtype=torch.float64).flatten()
    r = torch.as_tensor(np.asarray(ref.detach().cpu().double()) if isinstance(ref, torch.Tensor) else ref,
                        dtype=torch.float64).flatten()
    max_rel = float((g - r).abs().max() / r.abs().max().clamp_min(1e-300))
    cos = float(torch.dot(g, r) / (g.norm() * r.norm()).clamp_min(1e-300))
    return max_rel, cos


def assert_parity(loss, loss_ref, grads, grads_ref, what=""):
    le = loss_rel_err(loss, loss_ref)
    assert le <= LOSS_RTOL, f"{what}: loss rel err {le:.3e} > {LOSS_RTOL}"
    for name, (g, r) in zip(("grad0", "grad1"), zip(grads, grads_ref)):
        mr, cs = grad_errors(g, r)
        assert mr <= GRAD_MAX_REL, f"{what}: {name} max-rel {mr:.3e} > {GRAD_MAX_REL}"
        assert cs >= GRAD_COS_MIN, f"{what}: {name} cosine {cs:.6f} < {GRAD_COS_MIN}"
