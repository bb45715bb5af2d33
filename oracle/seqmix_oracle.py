"""CPU restatement (NumPy) of the reference's sequence-mixing patches.  TEST INFRASTRUCTURE ONLY.

causal_conv1d follows `_fast_call` of modal/fast_conv.py:14-31 (K shifted multiply-adds over a left-padded input)
and is pinned by golden vectors produced by running that function (tests/golden/make_golden_seqmix.py).
"""
from __future__ import annotations

import numpy as np

__all__ = ["causal_conv1d", "causal_conv1d_bwd", "recurrent_gated_delta_rule", "chunk_gated_delta_rule",
           "chunk_gated_delta_rule_bwd"]


def causal_conv1d(x, w):
  """y[b,t,c] = sum_j w[j,0,c] * x[b, t-(K-1)+j, c];  x [B,T,C], w [K,1,C] (modal/fast_conv.py:25-30)."""
  x = np.asarray(x, np.float32)
  w = np.asarray(w, np.float32)
  ks, t = w.shape[0], x.shape[1]
  xp = np.pad(x, ((0, 0), (ks - 1, 0), (0, 0)))
  y = xp[:, 0:t, :] * w[0, 0]
  for j in range(1, ks):
    y = y + xp[:, j:j + t, :] * w[j, 0]
  return y.astype(np.float32)


def causal_conv1d_bwd(g, x, w):
  """(dx, dw) of causal_conv1d: dx is the same sum run forwards in time over g, dw[j] = sum_{b,t} g * shifted x."""
  g = np.asarray(g, np.float32)
  x = np.asarray(x, np.float32)
  w = np.asarray(w, np.float32)
  ks, t = w.shape[0], x.shape[1]
  gp = np.pad(g, ((0, 0), (0, ks - 1), (0, 0)))
  xp = np.pad(x, ((0, 0), (ks - 1, 0), (0, 0)))
  dx = np.zeros_like(x)
  dw = np.zeros_like(w)
  for j in range(ks):
    dx += gp[:, ks - 1 - j:ks - 1 - j + t, :] * w[j, 0]
    dw[j, 0] = (g * xp[:, j:j + t, :]).sum(axis=(0, 1))
  return dx, dw


def _bf16(a):
  from .moe_oracle import bf16_round
  return bf16_round(np.asarray(a, np.float32))


def recurrent_gated_delta_rule(q, k, v, g, beta, initial_state=None):
  """The gated delta rule one token at a time, in float64: the definition the chunked form must reproduce.

    h <- h * exp(g_t);  v' = beta_t * (v_t - k_t^T h);  h <- h + k_t (x) v';  o_t = (q_t / sqrt(K))^T h

  q, k [B,S,H,K], v [B,S,H,V], g, beta [B,S,H]; state h [B,H,K,V].  Returns (o [B,S,H,V], final h)."""
  q, k, v, g, beta = (np.asarray(a, np.float64) for a in (q, k, v, g, beta))
  b, s, hh, kd = k.shape
  vd = v.shape[-1]
  h = np.zeros((b, hh, kd, vd)) if initial_state is None else np.asarray(initial_state, np.float64).copy()
  o = np.zeros((b, s, hh, vd))
  scale = 1.0 / np.sqrt(kd)
  for t in range(s):
    h = h * np.exp(g[:, t])[..., None, None]
    vn = beta[:, t][..., None] * (v[:, t] - np.einsum("bhk,bhkv->bhv", k[:, t], h))
    h = h + np.einsum("bhk,bhv->bhkv", k[:, t], vn)
    o[:, t] = np.einsum("bhk,bhkv->bhv", q[:, t] * scale, h)
  return o, h


def chunk_gated_delta_rule(q, k, v, g, beta, chunk_size=64, initial_state=None, inverse="solve"):
  """The chunked form, restating `fast_chunk_gated_delta_rule` (modal/gdn_fast.py:37-113) step by step with its
  dtype rules for compute_dtype = bfloat16: q, k, v, beta are bf16 values, q is scaled in bf16, products of two bf16
  arrays are rounded to bf16 (S, the in-chunk attention, u, w), everything that involves g or the state is float32.
  `inverse`: "solve" (triangular solve) or "neumann" (the product form of `_inv_unit_lower`, :21-34)."""
  f32 = np.float32
  q, k, v, beta = (_bf16(a) for a in (q, k, v, beta))
  g = np.asarray(g, f32)
  b, s, hh, kd = k.shape
  vd = v.shape[-1]
  q = _bf16(q * _bf16(f32(1.0) / np.sqrt(f32(kd))))
  pad = (-s) % chunk_size
  if pad:
    padf = lambda a: np.pad(a, ((0, 0), (0, pad)) + ((0, 0),) * (a.ndim - 2))
    q, k, v, g, beta = map(padf, (q, k, v, g, beta))
  n = q.shape[1] // chunk_size
  c = chunk_size
  chunked = lambda a: a.reshape(b, n, c, hh, -1).transpose(0, 1, 3, 2, 4)          # [B,N,H,C,*]
  q_c, k_c, v_c = chunked(q), chunked(k), chunked(v)
  g_c = g.reshape(b, n, c, hh).transpose(0, 1, 3, 2)
  beta_c = beta.reshape(b, n, c, hh).transpose(0, 1, 3, 2)
  gcs = np.cumsum(g_c, axis=-1, dtype=f32)
  k_beta = _bf16(k_c * beta_c[..., None])
  strict = np.tril(np.ones((c, c), bool), k=-1)
  s_mat = _bf16(k_beta @ k_c.swapaxes(-1, -2))
  decay = np.where(strict, gcs[..., :, None] - gcs[..., None, :], f32(-1e30))
  s_mat = np.where(strict, s_mat * np.exp(decay), f32(0)).astype(f32)
  eye = np.eye(c, dtype=f32)
  if inverse == "solve":
    a_mat = np.linalg.solve((eye + s_mat).astype(np.float64), np.broadcast_to(eye, s_mat.shape).astype(np.float64)).astype(f32)
  else:
    a_mat, p, m = eye - s_mat, s_mat, 2
    while m < c:
      p = p @ p
      a_mat = a_mat @ (eye + p)
      m *= 2
  v_beta = _bf16(v_c * beta_c[..., None])
  u = _bf16(a_mat @ v_beta)
  w = _bf16(a_mat @ (k_beta * np.exp(gcs)[..., None]))
  h = np.zeros((b, hh, kd, vd), f32) if initial_state is None else np.asarray(initial_state, f32).copy()
  incl = np.tril(np.ones((c, c), bool))
  o = np.zeros((b, n, hh, c, vd), f32)
  for i in range(n):
    gg = gcs[:, i]
    q_g = q_c[:, i] * np.exp(gg)[..., None]
    v_new = u[:, i] - w[:, i] @ h
    attn = _bf16(q_c[:, i] @ k_c[:, i].swapaxes(-1, -2))
    gd = np.where(incl, gg[..., :, None] - gg[..., None, :], f32(-1e30))
    attn = np.where(incl, attn * np.exp(gd), f32(0))
    o[:, i] = q_g @ h + attn @ v_new
    k_i = k_c[:, i] * np.exp(gg[..., -1, None] - gg)[..., None]
    h = h * np.exp(gg[..., -1, None, None]) + k_i.swapaxes(-1, -2) @ v_new
  o = o.transpose(0, 1, 3, 2, 4).reshape(b, -1, hh, vd)[:, :s]
  return o.astype(f32), h.astype(f32)


def chunk_gated_delta_rule_bwd(q, k, v, g, beta, do, dh_final=None, initial_state=None, chunk_size=64):
  """Gradient of `chunk_gated_delta_rule` (the solve form) written out by hand, in float64.

  The reference has no backward of its own: JAX differentiates `fast_chunk_gated_delta_rule` (modal/gdn_fast.py:37-113),
  and a cast to bfloat16 differentiates as the identity.  So the forward values below carry the forward pass's
  roundings and the derivative ignores them.  tests/test_seqmix.py pins this function against torch autograd of a
  differentiable restatement of the forward (roundings straight-through), which in turn equals the forward oracle.
  Returns (dq, dk, dv, dg, dbeta, dh0)."""
  f = np.float64
  b, s, hh, kd = np.shape(k)
  c = chunk_size
  q, k, v, beta = (_bf16(a).astype(f) for a in (q, k, v, beta))
  g = np.asarray(g, np.float32).astype(f)
  do = np.asarray(do, f)
  scale = f(_bf16(np.float32(1.0) / np.sqrt(np.float32(kd))).reshape(-1)[0])
  pad = (-s) % c
  if pad:
    padf = lambda a: np.pad(a, ((0, 0), (0, pad)) + ((0, 0),) * (a.ndim - 2))
    q, k, v, g, beta, do = map(padf, (q, k, v, g, beta, do))
  n = q.shape[1] // c
  chunked = lambda a: a.reshape(b, n, c, hh, -1).transpose(0, 1, 3, 2, 4)      # [B,N,H,C,*]
  qs = _bf16(chunked(q) * scale).astype(f)
  k_c, v_c, do_c = chunked(k), chunked(v), chunked(do)
  g_c = g.reshape(b, n, c, hh).transpose(0, 1, 3, 2)
  beta_c = beta.reshape(b, n, c, hh).transpose(0, 1, 3, 2)
  gcs = np.cumsum(g_c.astype(np.float32), -1, dtype=np.float32).astype(f)
  strict = np.tril(np.ones((c, c), bool), -1)
  incl = np.tril(np.ones((c, c), bool))
  kb = _bf16(k_c * beta_c[..., None]).astype(f)
  vb = _bf16(v_c * beta_c[..., None]).astype(f)
  p_mat = _bf16(kb @ k_c.swapaxes(-1, -2)).astype(f)
  d_mat = np.exp(np.where(incl, gcs[..., :, None] - gcs[..., None, :], 0.0))
  s_mat = np.where(strict, p_mat * d_mat, 0.0)
  a_mat = np.linalg.solve(np.eye(c) + s_mat, np.broadcast_to(np.eye(c), s_mat.shape).copy())
  e_vec = np.exp(gcs)
  kg = kb * e_vec[..., None]
  u = _bf16(a_mat @ vb).astype(f)
  w = _bf16(a_mat @ kg).astype(f)
  attn = np.where(incl, _bf16(qs @ k_c.swapaxes(-1, -2)).astype(f) * d_mat, 0.0)
  # the state at the start of every chunk
  h = np.zeros((b, hh, kd, v.shape[-1]), f) if initial_state is None else np.asarray(initial_state, f).copy()
  states = []
  for i in range(n):
    states.append(h)
    vn = u[:, i] - w[:, i] @ h
    k_dec = k_c[:, i] * np.exp(gcs[:, i, :, -1, None] - gcs[:, i])[..., None]
    h = h * np.exp(gcs[:, i, :, -1])[..., None, None] + k_dec.swapaxes(-1, -2) @ vn
  dh = np.zeros_like(h) if dh_final is None else np.asarray(dh_final, f).copy()
  dqs, dk, dvb, dkb, dgcs = (np.zeros_like(a) for a in (qs, k_c, vb, kb, gcs))
  for i in reversed(range(n)):
    h_in, gg = states[i], gcs[:, i]
    gl, e_i = gg[..., -1], e_vec[:, i]
    vn = u[:, i] - w[:, i] @ h_in
    e_dk = np.exp(gl[..., None] - gg)
    k_dec = k_c[:, i] * e_dk[..., None]
    q_e = qs[:, i] * e_i[..., None]
    d_o = do_c[:, i]
    # the recurrence
    dvn = attn[:, i].swapaxes(-1, -2) @ d_o + k_dec @ dh
    dattn = np.where(incl, d_o @ vn.swapaxes(-1, -2), 0.0)
    dq_e = d_o @ h_in.swapaxes(-1, -2)
    dk_dec = vn @ dh.swapaxes(-1, -2)
    dh_in = q_e.swapaxes(-1, -2) @ d_o + dh * np.exp(gl)[..., None, None] - w[:, i].swapaxes(-1, -2) @ dvn
    dgc = (dq_e * q_e).sum(-1) - (dk_dec * k_dec).sum(-1)
    dgc[..., -1] += (dh * h_in).sum((-1, -2)) * np.exp(gl) + (dk_dec * k_dec).sum((-1, -2))
    dqs[:, i] += dq_e * e_i[..., None]
    dk[:, i] += dk_dec * e_dk[..., None]
    dw = -dvn @ h_in.swapaxes(-1, -2)
    # the in-chunk attention
    gmat = dattn * attn[:, i]
    dgc += gmat.sum(-1) - gmat.sum(-2)
    d_qk = dattn * d_mat[:, i]
    dqs[:, i] += d_qk @ k_c[:, i]
    dk[:, i] += d_qk.swapaxes(-1, -2) @ qs[:, i]
    # u = A vb, w = A kg
    a_i = a_mat[:, i]
    d_a = dvn @ vb[:, i].swapaxes(-1, -2) + dw @ kg[:, i].swapaxes(-1, -2)
    dvb[:, i] += a_i.swapaxes(-1, -2) @ dvn
    dkg = a_i.swapaxes(-1, -2) @ dw
    dkb[:, i] += dkg * e_i[..., None]
    dgc += (dkg * kg[:, i]).sum(-1)
    # A = (I + S)^-1, S = strict(P D)
    d_s = np.where(strict, -(a_i.swapaxes(-1, -2) @ d_a @ a_i.swapaxes(-1, -2)), 0.0)
    gmat = d_s * s_mat[:, i]
    dgc += gmat.sum(-1) - gmat.sum(-2)
    d_p = d_s * d_mat[:, i]
    dkb[:, i] += d_p @ k_c[:, i]
    dk[:, i] += d_p.swapaxes(-1, -2) @ kb[:, i]
    dgcs[:, i] = dgc
    dh = dh_in
  dk += dkb * beta_c[..., None]
  dbeta = (dkb * k_c).sum(-1) + (dvb * v_c).sum(-1)
  dv = dvb * beta_c[..., None]
  dg = np.flip(np.cumsum(np.flip(dgcs, -1), -1), -1)
  rows = lambda a: a.transpose(0, 1, 3, 2, 4).reshape(b, n * c, hh, -1)[:, :s]
  vecs = lambda a: a.transpose(0, 1, 3, 2).reshape(b, n * c, hh)[:, :s]
  return rows(dqs * scale), rows(dk), rows(dv), vecs(dg), vecs(dbeta), dh
