"""Generates tests/golden/moe_mlp_*.npz from the reference's own PyTorch MoE layer.

Run where the reference tree is present:

    python tests/golden/make_golden.py [/path/to/reference]

It imports `MoEMLP` from
test/dataflow_models/correctness_compare/test_moe/moe_model_flash2.py:354-450 of the
reference, runs forward + autograd backward on CPU for small seeded shapes and stores inputs
and results (bf16 tensors as uint16 bit patterns). The router is run in fp32 (the layer's
`router_dtype` argument) from bf16-representable weights, which is the precision the CUDA
path here uses for logits. The committed .npz files are what the tests read; the reference
tree is not needed to run the tests.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

CASES = {
    # name: (T, d, E, k, f, seed)
    "moe_mlp_small": (96, 128, 8, 2, 64, 1234),
    "moe_mlp_k4": (80, 64, 16, 4, 96, 4321),
    "moe_mlp_e64k8": (72, 64, 64, 8, 32, 777),   # the benchmark's routing shape: 64 experts, top-8 (9 rows per expert)
}


def bits(t):
    return t.detach().to(torch.bfloat16).contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def main():
    if len(sys.argv) < 2 and not os.environ.get("REFERENCE_ROOT"):
        sys.exit("usage: make_golden.py <path of the reference checkout>   (or set REFERENCE_ROOT)")
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ["REFERENCE_ROOT"]
    sys.path.insert(0, os.path.join(ref_root, "test/dataflow_models/correctness_compare/test_moe"))
    import moe_model_flash2 as ref  # noqa: E402

    for name, (T, d, E, k, f, seed) in CASES.items():
        g = torch.Generator().manual_seed(seed)

        def rnd(*shape, std=1.0):
            return (torch.randn(*shape, generator=g) * std).to(torch.bfloat16)

        X = rnd(T, d)
        dOut = rnd(T, d)
        Wr = rnd(E, d, std=0.3)
        W1 = rnd(E, f, d, std=0.08)
        W3 = rnd(E, f, d, std=0.08)
        W2 = rnd(E, d, f, std=0.08)

        layer = ref.MoEMLP(E, k, d, f, layer_id=0, router_dtype=torch.float32, expert_dtype=torch.bfloat16)
        with torch.no_grad():
            layer.gate.weight.copy_(Wr.float())
            for e in range(E):
                layer.experts[e].gate_proj.weight.copy_(W1[e])
                layer.experts[e].up_proj.weight.copy_(W3[e])
                layer.experts[e].down_proj.weight.copy_(W2[e])
        x = X.clone().view(1, T, d).requires_grad_(True)
        out, logits = layer(x, 0)
        out.backward(dOut.view(1, T, d))

        # routing as the layer computes it (moe_model_flash2.py:405-407)
        rw = torch.softmax(logits, dim=1, dtype=torch.float)
        rw, sel = torch.topk(rw, k, dim=-1)
        rw = rw / rw.sum(dim=-1, keepdim=True)

        np.savez_compressed(
            os.path.join(HERE, name + ".npz"),
            shape=np.array([T, d, E, k, f], np.int32),
            X=bits(X), dOut=bits(dOut), Wr=bits(Wr), W1=bits(W1), W3=bits(W3), W2=bits(W2),
            logits=logits.detach().float().numpy(),
            selected=sel.numpy().astype(np.int32),
            routing_weights=rw.detach().numpy().astype(np.float32),
            out=bits(out.view(T, d)),
            dX=bits(x.grad.view(T, d)),
            dWr=layer.gate.weight.grad.float().numpy(),
            dW1=bits(torch.stack([layer.experts[e].gate_proj.weight.grad for e in range(E)])),
            dW3=bits(torch.stack([layer.experts[e].up_proj.weight.grad for e in range(E)])),
            dW2=bits(torch.stack([layer.experts[e].down_proj.weight.grad for e in range(E)])),
        )
        print("wrote", name, "out absmax", float(out.abs().max()))


if __name__ == "__main__":
    main()
