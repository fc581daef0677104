"""ctypes binding of the CPU oracle (oracle/moe_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and by
bench.py's cpu_baseline / reference legs. The product package never imports it.

All tensors are numpy arrays; bf16 travels as uint16 bit patterns. The layer
functions at the bottom restate the order in which the reference's MoE block
submits ops (libdataflowmodels/src/transformer/src/dataflow_transformer.c:
forward 2588-2986, backward-x 3386-3719, backward-w 4060-4185).
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")
DT_FP32, DT_BF16 = 3, 5


def reference_root():
    """The reference checkout: $REFERENCE_ROOT, else a directory named `reference` beside this repository."""
    return os.environ.get("REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")


def build(force=False):
    if force or not os.path.exists(_LIB_PATH) or (
        os.path.getmtime(_LIB_PATH) < max(os.path.getmtime(os.path.join(_HERE, n)) for n in ("moe_oracle.c", "block_oracle.c"))
    ):
        subprocess.check_call(["make", "-C", _HERE, "liboracle.so"], stdout=subprocess.DEVNULL)
    if os.path.isdir(reference_root()):
        # the reference's own kernels (cubins) and host submitters, compiled from its sources in place
        subprocess.call(["make", "-C", _HERE, "ref", "dropin", "REFERENCE_ROOT=" + reference_root()],
                        stdout=subprocess.DEVNULL)


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.orc_num_threads.restype = C.c_int
        _lib.orc_matmul.restype = C.c_int
    return _lib


def _p(a):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(C.c_void_p)


def num_threads():
    return lib().orc_num_threads()


def use_all_cores():
    """Makes the oracle's OpenMP loops use every core this process may run on, whatever OMP_NUM_THREADS says (process
    launchers set it to 1). Returns the thread count now in use."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().orc_set_num_threads(C.c_int(n))
    return num_threads()


# ---- bf16 helpers -----------------------------------------------------------

def to_bf16(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().orc_f32_to_bf16(_p(x), _p(out), C.c_int64(x.size))
    return out


def to_f32(x):
    x = np.ascontiguousarray(x, dtype=np.uint16)
    out = np.empty(x.shape, dtype=np.float32)
    lib().orc_bf16_to_f32(_p(x), _p(out), C.c_int64(x.size))
    return out


def normal_bf16(shape, seed, mean=0.0, std=1.0):
    out = np.empty(shape, dtype=np.uint16)
    lib().orc_fill_normal_bf16(_p(out), C.c_int64(out.size), C.c_uint64(seed), C.c_float(mean), C.c_float(std))
    return out


def normal_f32(shape, seed, mean=0.0, std=1.0):
    out = np.empty(shape, dtype=np.float32)
    lib().orc_fill_normal_f32(_p(out), C.c_int64(out.size), C.c_uint64(seed), C.c_float(mean), C.c_float(std))
    return out


# ---- ops ----------------------------------------------------------------------

def select_experts(logits, top_k):
    """Returns weights[T,k] f32, chosen[T,k] u16, counts[E+1] i32, cumsum[E] i32 (exclusive), host_counts[E]."""
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    T, E = logits.shape
    w = np.empty((T, top_k), np.float32)
    ch = np.empty((T, top_k), np.uint16)
    counts = np.zeros(E + 1, np.int32)
    cumsum = np.zeros(E, np.int32)
    host = np.zeros(E, np.int32)
    lib().orc_select_experts_f32(T, E, top_k, _p(logits), _p(w), _p(ch), _p(counts), _p(cumsum), _p(host))
    return w, ch, counts, cumsum, host


def build_expert_mapping(chosen, n_experts, cumsum_excl):
    """Returns expert_mapping[R], token_mapping[T,k], inclusive cumsum[E]."""
    T, k = chosen.shape
    cumsum = np.array(cumsum_excl, dtype=np.int32, copy=True)
    em = np.full(T * k, -1, np.int32)
    tm = np.empty((T, k), np.int32)
    lib().orc_build_expert_mapping(T, n_experts, k, _p(np.ascontiguousarray(chosen)), _p(cumsum), _p(em), _p(tm))
    return em, tm, cumsum


def prepare_experts(X, token_mapping, zone=None):
    T, d = X.shape
    k = token_mapping.shape[1]
    if zone is None:
        zone = np.zeros((T * k, d), np.uint16)
    lib().orc_prepare_experts(T, d, k, _p(X), _p(token_mapping), _p(zone))
    return zone


def prepare_expert_zone(X, expert_id, counts, cumsum_incl, expert_mapping):
    d = X.shape[1]
    zone = np.zeros((int(counts[expert_id]), d), np.uint16)
    lib().orc_prepare_expert_zone(d, _p(X), expert_id, _p(counts), _p(cumsum_incl), _p(expert_mapping), _p(zone))
    return zone


def merge_experts(zone, token_mapping, weights, X_combined):
    """In place on X_combined ([T,d] uint16). weights may be None (all 1.0)."""
    T, d = X_combined.shape
    k = token_mapping.shape[1]
    lib().orc_merge_experts(T, d, k, _p(zone), _p(token_mapping), _p(weights), _p(X_combined))
    return X_combined


def merge_expert_result(zone_e, expert_id, cumsum_incl, expert_mapping, weights, chosen, X_combined):
    n, d = zone_e.shape
    k = chosen.shape[1]
    lib().orc_merge_expert_result(n, d, k, _p(zone_e), expert_id, _p(cumsum_incl), _p(expert_mapping),
                                  _p(weights), _p(chosen), _p(X_combined))
    return X_combined


def swiglu(x1, x3):
    out = np.empty_like(x1)
    r, c = x1.shape
    lib().orc_swiglu(r, c, _p(x1), _p(x3), _p(out))
    return out


def swiglu_bwd_x(x1, x3, dy):
    r, c = x1.shape
    d1, d3 = np.empty_like(x1), np.empty_like(x1)
    lib().orc_swiglu_bwd_x(r, c, _p(x1), _p(x3), _p(dy), _p(d1), _p(d3))
    return d1, d3


def router_bwd_x(n_e, d, E, k, expert_id, cumsum_incl, expert_mapping, chosen, weights,
                 expert_out, upstream_dX, dX_routed, dX_expert_out):
    lib().orc_router_bwd_x(n_e, d, E, k, expert_id, _p(cumsum_incl), _p(expert_mapping), _p(chosen), _p(weights),
                           _p(expert_out), _p(upstream_dX), _p(dX_routed), _p(dX_expert_out))


def router_gate_bwd_x(chosen, weights, dX_routed):
    T, E = dX_routed.shape
    lib().orc_router_gate_bwd_x(T, E, chosen.shape[1], _p(chosen), _p(weights), _p(dX_routed))
    return dX_routed


def _dt(a):
    return DT_FP32 if a.dtype == np.float32 else DT_BF16


def matmul(ta, tb, M, K, N, alpha, beta, A, B, Cm, D):
    """Column-major D[MxN] = alpha*op(A)*op(B) + beta*C (reference matmul semantics). D is written in place."""
    rc = lib().orc_matmul(_dt(A), _dt(B), _dt(Cm) if Cm is not None else 0, _dt(D), ta, tb, M, K, N,
                          C.c_float(alpha), C.c_float(beta), _p(A), _p(B), _p(Cm), _p(D))
    assert rc == 0
    return D


def linear_fwd(X, W, out_dtype=np.uint16):
    """Row-major Y[rows,out] = X[rows,in] . W[out,in]^T  (reference form transa=1, transb=0, M=out, K=in, N=rows)."""
    rows, kin = X.shape
    out = W.shape[0]
    Y = np.empty((rows, out), out_dtype)
    return matmul(1, 0, out, kin, rows, 1.0, 0.0, W, X, None, Y)


def linear_dgrad(dY, W, accumulate_into=None):
    """Row-major dX[rows,in] (+)= dY[rows,out] . W[out,in]  (transa=0, transb=0, M=in, K=out, N=rows)."""
    rows, out = dY.shape
    kin = W.shape[1]
    if accumulate_into is None:
        D = np.empty((rows, kin), np.uint16)
        return matmul(0, 0, kin, out, rows, 1.0, 0.0, W, dY, None, D)
    return matmul(0, 0, kin, out, rows, 1.0, 1.0, W, dY, accumulate_into, accumulate_into)


def linear_wgrad(X, dY, dW):
    """Row-major dW[out,in] += dY[rows,out]^T . X[rows,in]  (transa=0, transb=1, M=in, K=rows, N=out)."""
    rows, kin = X.shape
    out = dY.shape[1]
    return matmul(0, 1, kin, rows, out, 1.0, 1.0, X, dY, dW, dW)


# ---- the layer, in the reference block's op order -------------------------------

def moe_forward(Xn, Wr, W1, W3, W2, top_k, residual=None, logits=None):
    """One MoE layer forward. Xn [T,d] bf16; Wr [E,d]; W1,W3 [E,f,d]; W2 [E,d,f] (all uint16 bf16 bits).

    logits may be supplied (fp32 [T,E]) to bypass the router GEMM. Returns a dict with every
    intermediate the backward needs and `out` = residual + combined expert outputs.
    """
    T, d = Xn.shape
    E = Wr.shape[0]
    if logits is None:
        logits = linear_fwd(Xn, Wr, out_dtype=np.float32)
    w, chosen, counts, cumsum_excl, host_counts = select_experts(logits, top_k)
    em, tm, cumsum_incl = build_expert_mapping(chosen, E, cumsum_excl)
    zone = prepare_experts(Xn, tm)
    f = W1.shape[1]
    R = T * top_k
    x1 = np.zeros((R, f), np.uint16)
    x3 = np.zeros((R, f), np.uint16)
    Y = np.zeros((R, d), np.uint16)
    for e in range(E):
        n = int(host_counts[e])
        if n == 0:
            continue
        b = int(cumsum_excl[e])
        z = zone[b:b + n]
        x1[b:b + n] = linear_fwd(z, W1[e])
        x3[b:b + n] = linear_fwd(z, W3[e])
        h = swiglu(x1[b:b + n], x3[b:b + n])
        Y[b:b + n] = linear_fwd(h, W2[e])
    out = np.zeros((T, d), np.uint16) if residual is None else residual.copy()
    merge_experts(Y, tm, w, out)
    return dict(logits=logits, weights=w, chosen=chosen, counts=counts, cumsum_excl=cumsum_excl,
                cumsum_incl=cumsum_incl, host_counts=host_counts, expert_mapping=em, token_mapping=tm,
                zone=zone, x1=x1, x3=x3, Y=Y, out=out)


def moe_backward(Xn, Wr, W1, W3, W2, top_k, fwd, dOut, grads=None):
    """Backward of one MoE layer in the reference's op order (bwd_x then bwd_w).

    grads: optional dict of bf16 accumulators dW1,dW3 [E,f,d], dW2 [E,d,f], dWr [E,d] (accumulated into, like the
    reference's beta=1 matmuls); zero-initialised when absent. Returns dict with dXn, dlogits (bf16 [T,E]), dx1,
    dx3, dZ and the weight gradients.
    """
    T, d = Xn.shape
    E, f = W1.shape[0], W1.shape[1]
    R = T * top_k
    if grads is None:
        grads = dict(dW1=np.zeros_like(W1), dW3=np.zeros_like(W3), dW2=np.zeros_like(W2), dWr=np.zeros_like(Wr))
    em, tm, chosen, w = fwd["expert_mapping"], fwd["token_mapping"], fwd["chosen"], fwd["weights"]
    cumsum_incl, host_counts, cumsum_excl = fwd["cumsum_incl"], fwd["host_counts"], fwd["cumsum_excl"]
    dX_routed = np.zeros((T, E), np.uint16)
    zone = np.zeros((R, d), np.uint16)
    dx1 = np.zeros((R, f), np.uint16)
    dx3 = np.zeros((R, f), np.uint16)
    hs = np.zeros((R, f), np.uint16)
    for e in range(E):
        n = int(host_counts[e])
        if n == 0:
            continue
        b = int(cumsum_excl[e])
        h = swiglu(fwd["x1"][b:b + n], fwd["x3"][b:b + n])  # recompute (3494-3516)
        hs[b:b + n] = h
        y = linear_fwd(h, W2[e])
        ze = np.ascontiguousarray(zone[b:b + n])
        router_bwd_x(n, d, E, top_k, e, cumsum_incl, em, chosen, w, y, dOut, dX_routed, ze)
        zone[b:b + n] = ze  # now dY = w * dOut rows
        linear_wgrad(h, ze, grads["dW2"][e])  # dW2[d][f] += dY^T h   (3548-3560)
        dh = linear_dgrad(ze, W2[e])  # [n,f]                         (3568-3579)
        d1, d3 = swiglu_bwd_x(fwd["x1"][b:b + n], fwd["x3"][b:b + n], dh)
        dx1[b:b + n], dx3[b:b + n] = d1, d3
        dz = linear_dgrad(d1, W1[e])  # (3601-3612)
        dz = linear_dgrad(d3, W3[e], accumulate_into=dz)  # beta=1 in place (3614-3625)
        zone[b:b + n] = dz
    dXn = np.zeros((T, d), np.uint16)
    merge_experts(zone, tm, None, dXn)  # un-permute (3666-3682)
    router_gate_bwd_x(chosen, w, dX_routed)  # (3695-3704)
    linear_dgrad(dX_routed, Wr, accumulate_into=dXn)  # (3707-3719)
    # bwd_w (4062-4185)
    zx = prepare_experts(Xn, tm)
    for e in range(E):
        n = int(host_counts[e])
        if n == 0:
            continue
        b = int(cumsum_excl[e])
        linear_wgrad(zx[b:b + n], dx1[b:b + n], grads["dW1"][e])
        linear_wgrad(zx[b:b + n], dx3[b:b + n], grads["dW3"][e])
    linear_wgrad(Xn, dX_routed, grads["dWr"])
    return dict(dXn=dXn, dlogits=dX_routed, dx1=dx1, dx3=dx3, dZ=zone, h=hs, **grads)


# ---- block ops (oracle/block_oracle.c): numpy in, numpy out; bf16 as uint16 bit patterns -------------------------
def rms_norm(w, X, eps):
    n_rows, n_cols = X.shape
    out, rms = np.empty_like(X), np.empty(n_rows, np.float32)
    lib().orc_rms_norm_bf16(n_rows, n_cols, C.c_float(eps), _p(w), _p(X), _p(out), _p(rms))
    return out, rms


def rms_norm_recompute(w, rms, X):
    out = np.empty_like(X)
    lib().orc_rms_norm_recompute_bf16(X.shape[0], X.shape[1], _p(w), _p(rms), _p(X), _p(out))
    return out


def rms_norm_bwd_x(rms, w, X, up, dX, want_x_out=False):
    """Accumulates into a copy of dX; returns (dX_new, X_out or None)."""
    dX = dX.copy()
    x_out = np.empty_like(X) if want_x_out else None
    lib().orc_rms_norm_bwd_x_bf16(X.shape[0], X.shape[1], _p(rms), _p(w), _p(X), _p(up), _p(dX), _p(x_out))
    return dX, x_out


def rms_norm_bwd_w(rms, X, up, dW):
    dW = dW.copy()
    lib().orc_rms_norm_bwd_w_bf16(X.shape[0], X.shape[1], _p(rms), _p(X), _p(up), _p(dW))
    return dW


def rope(head_dim, num_kv_heads, theta, seq_positions, X_q, X_k=None, backward=False):
    X_q = X_q.copy()
    X_k = None if X_k is None else X_k.copy()
    fn = lib().orc_rope_bwd_x_bf16 if backward else lib().orc_rope_bf16
    fn(X_q.shape[0], X_q.shape[1], head_dim, num_kv_heads, int(theta), _p(np.ascontiguousarray(seq_positions, np.int32)),
       _p(X_q), _p(X_k))
    return X_q, X_k


def softmax(X):
    out = np.empty_like(X)
    lib().orc_softmax_bf16(X.shape[0], X.shape[1], _p(X), _p(out))
    return out


def cross_entropy_loss(p, labels):
    """Returns (p with 1 subtracted at the labels, loss_vec of n_rows + 1 entries with the average in the last)."""
    p = p.copy()
    n = p.shape[0]
    loss = np.zeros(n + 1, np.float32)
    lib().orc_cross_entropy_loss_bf16(n, p.shape[1], _p(p), _p(np.ascontiguousarray(labels, np.uint32)), _p(loss))
    lib().orc_set_average_loss(n, _p(loss))
    return p, loss


def adamw_step(step, lr, b1, b2, wd, eps, param, grad, mean, var):
    param, mean, var = param.copy(), mean.copy(), var.copy()
    f = C.c_float
    lib().orc_adamw_step_bf16(C.c_uint64(param.size), step, f(lr), f(b1), f(b2), f(wd), f(eps), _p(param), _p(grad), _p(mean),
                              _p(var))
    return param, mean, var


def sort_tokens(token_ids):
    """The reference's host-side preparation for the embedding ops (sorted ids, their positions, start of each unique
    id's run, with one closing entry)."""
    token_ids = np.asarray(token_ids, np.uint32)
    order = np.argsort(token_ids, kind="stable").astype(np.uint32)
    sorted_ids = token_ids[order]
    starts = np.flatnonzero(np.concatenate([[True], sorted_ids[1:] != sorted_ids[:-1]])).astype(np.uint32)
    return sorted_ids, order, np.concatenate([starts, [len(token_ids)]]).astype(np.uint32)


def embedding_table(sorted_ids, mapping, starts, table, n_tokens):
    out = np.zeros((n_tokens, table.shape[1]), np.uint16)
    lib().orc_embedding_table_bf16(len(starts) - 1, table.shape[1], _p(sorted_ids), _p(mapping), _p(starts), _p(table), _p(out))
    return out


def embedding_table_bwd_w(sorted_ids, mapping, starts, grad_stream, grad_table):
    grad_table = grad_table.copy()
    lib().orc_embedding_table_bwd_w_bf16(len(starts) - 1, grad_table.shape[1], _p(sorted_ids), _p(mapping), _p(starts),
                                         _p(grad_stream), _p(grad_table))
    return grad_table


def attention_fwd(q_off, q_len, k_off, k_len, Hq, Hkv, hd, Q, K, V, causal=True):
    """Returns (O bf16 bits [total_q, Hq*hd], lse float32 [Hq, total_q])."""
    O = np.zeros_like(Q)
    lse = np.zeros((Hq, Q.shape[0]), np.float32)
    ia = lambda a: _p(np.ascontiguousarray(a, np.int32))
    lib().orc_attention_fwd_bf16(len(q_len), Q.shape[0], ia(q_off), ia(q_len), ia(k_off), ia(k_len), Hq, Hkv, hd, _p(Q), _p(K),
                                 _p(V), _p(O), _p(lse), int(bool(causal)))
    return O, lse


def attention_bwd(q_off, q_len, k_off, k_len, Hq, Hkv, hd, Q, K, V, O, lse, dO, causal=True):
    dQ, dK, dV = np.zeros_like(Q), np.zeros_like(K), np.zeros_like(V)
    ia = lambda a: _p(np.ascontiguousarray(a, np.int32))
    lib().orc_attention_bwd_bf16(len(q_len), Q.shape[0], K.shape[0], ia(q_off), ia(q_len), ia(k_off), ia(k_len), Hq, Hkv, hd,
                                 _p(Q), _p(K), _p(V), _p(O), _p(lse), _p(dO), _p(dQ), _p(dK), _p(dV), int(bool(causal)))
    return dQ, dK, dV
