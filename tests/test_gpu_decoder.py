"""GPU: a small MoE decoder (2 layers, d=64, 4 query / 2 kv heads of 16, 8 experts top-2, ffn 32, vocabulary 256,
two packed sequences) through ml_dataflow_b200.decoder - every op on the sm_100a kernels - against the same model in
float32 torch autograd with the routing held fixed (the experts each token chose on the GPU). Loss and every kind of
gradient (embedding, projections, norms, router, experts, head) are compared as relative Frobenius errors: the GPU
path rounds to bf16 after every op, the reference never does. Then one AdamW step must move every parameter. Run twice:
with every block going through the C driver (b200_transformer_block_fwd / _bwd) and op by op from Python."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _reference(dec, token_ids, labels, seq_lens):
    import torch

    c = dec.cfg
    f32 = lambda t: t.detach().float().clone().requires_grad_(True)
    P = [{k: f32(v) for k, v in L.items()} for L in dec.layers]
    embed, final_norm, head = f32(dec.embed), f32(dec.final_norm), f32(dec.head)

    def rms(x, w):
        return x * torch.rsqrt((x * x).mean(dim=1, keepdim=True) + c.eps) * w

    pos = torch.cat([torch.arange(n) for n in seq_lens]).to(token_ids.device).float()
    inv = c.theta ** (-torch.arange(0, c.head_dim, 2, device=token_ids.device).float() / c.head_dim)
    ang = pos[:, None] * inv[None, :]
    cos, sin = torch.cos(ang), torch.sin(ang)

    def rope(t, heads):
        t = t.view(t.shape[0], heads, c.head_dim // 2, 2)
        e, o = t[..., 0], t[..., 1]
        return torch.stack([cos[:, None] * e - sin[:, None] * o, cos[:, None] * o + sin[:, None] * e], dim=-1).reshape(
            t.shape[0], heads * c.head_dim)

    x = embed[token_ids.long()]
    group = c.n_heads // c.n_kv_heads
    for li, L in enumerate(P):
        xn = rms(x, L["attn_norm"])
        q, k, v = rope(xn @ L["wq"].T, c.n_heads), rope(xn @ L["wk"].T, c.n_kv_heads), xn @ L["wv"].T
        attn = torch.zeros_like(q)
        off = 0
        for n in seq_lens:
            for h in range(c.n_heads):
                g = h // group
                qs = q[off:off + n, h * c.head_dim:(h + 1) * c.head_dim]
                ks = k[off:off + n, g * c.head_dim:(g + 1) * c.head_dim]
                vs = v[off:off + n, g * c.head_dim:(g + 1) * c.head_dim]
                sc = (qs @ ks.T) / np.sqrt(c.head_dim)
                sc = sc.masked_fill(torch.triu(torch.ones(n, n, dtype=torch.bool, device=sc.device), 1), float("-inf"))
                attn[off:off + n, h * c.head_dim:(h + 1) * c.head_dim] = torch.softmax(sc, dim=1) @ vs
            off += n
        x_mid = x + attn @ L["wo"].T
        xn2 = rms(x_mid, L["ffn_norm"])
        chosen = (dec.saved[li]["moe"].chosen.view(torch.int16).long() & 0xFFFF)  # [T, k], routing held fixed
        logits = xn2 @ L["router"].T
        gate = torch.softmax(torch.gather(logits, 1, chosen), dim=1)
        out = x_mid.clone()
        for j in range(c.top_k):
            e = chosen[:, j]
            a = torch.einsum("td,tfd->tf", xn2, L["W1"][e])
            b = torch.einsum("td,tfd->tf", xn2, L["W3"][e])
            y = torch.einsum("tf,tdf->td", torch.nn.functional.silu(a) * b, L["W2"][e])
            out = out + gate[:, j:j + 1] * y
        x = out
    logits = rms(x, final_norm) @ head.T
    loss = torch.nn.functional.cross_entropy(logits, labels.long(), reduction="sum")
    loss.backward()
    return loss.item() / token_ids.numel(), P, embed, final_norm, head


@pytest.mark.parametrize("c_blocks", [True, False], ids=["c_block_driver", "op_by_op"])
def test_decoder_step_against_float32_autograd(c_blocks):
    import torch

    from gpu_util import require_b200

    require_b200()
    from ml_dataflow_b200 import ops
    from ml_dataflow_b200.decoder import Decoder, DecoderConfig

    cfg = DecoderConfig(n_layers=2, d=64, n_heads=4, n_kv_heads=2, head_dim=16, n_experts=8, top_k=2, ffn=32, vocab=256,
                        theta=10000)
    seq_lens = [40, 56]
    T = sum(seq_lens)
    dec = Decoder(cfg, T, max(seq_lens), seed=3, std=0.1, c_blocks=c_blocks)
    if c_blocks:
        # the C driver writes the blocks' weight gradients (overwrite mode): whatever the buffers held must not matter
        for G in dec.grads:
            for g_ in G.values():
                g_.fill_(3.0)
    g = torch.Generator(device="cuda").manual_seed(5)
    tokens = torch.randint(0, cfg.vocab, (T,), generator=g, device="cuda", dtype=torch.int32)
    tokens[:10] = tokens[0]  # a repeated token for the embedding backward
    labels = torch.randint(0, cfg.vocab, (T,), generator=g, device="cuda", dtype=torch.int32)
    loss = dec.forward(tokens, labels, seq_lens)
    dec.backward()
    torch.cuda.synchronize()
    assert ops.gemm_status() == 0
    ref_loss, P, embed, final_norm, head = _reference(dec, tokens, labels, seq_lens)
    assert abs(loss.item() - ref_loss) < 2e-2 * abs(ref_loss), (loss.item(), ref_loss)

    def rel(got, ref):
        return ((got.float() - ref).norm() / (ref.norm() + 1e-30)).item()

    errs = {"embed": rel(dec.g_embed, embed.grad), "final_norm": rel(dec.g_final_norm, final_norm.grad),
            "head": rel(dec.g_head, head.grad)}
    for li in range(cfg.n_layers):
        for name in Decoder.PARAMS:
            errs[f"layer{li}.{name}"] = rel(dec.grads[li][name], P[li][name].grad)
    bad = {k: round(v, 4) for k, v in errs.items() if not v < 6e-2}
    assert not bad, f"gradients off: {bad}; all: { {k: round(v, 4) for k, v in errs.items()} }"
    # one optimizer step moves every parameter tensor and keeps it finite (a step large enough to clear half a bf16 ulp
    # of the norm weights, which start at 1.0)
    before = [p.clone() for p, _ in dec._all_params()]
    dec.adamw_step(lr=5e-2)
    torch.cuda.synchronize()
    for b, (p, _) in zip(before, dec._all_params()):
        assert torch.isfinite(p.float()).all() and not torch.equal(b, p)
    assert dec.num_params() == sum(b.numel() for b in before)
