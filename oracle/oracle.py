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
        os.path.getmtime(_LIB_PATH) < os.path.getmtime(os.path.join(_HERE, "moe_oracle.c"))
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
