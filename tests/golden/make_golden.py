"""Generates tests/golden/*.npz with torch's CPU kernels (an implementation independent of
oracle/ixk_oracle.py): the CPU oracle is checked against these files, and so are the CUDA
kernels.  The reference itself cannot produce vectors here (its kernels need a SYCL
toolchain and XeTLA / oneDNN), so these stand in for them.

    python tests/golden/make_golden.py            # all files
    python tests/golden/make_golden.py backward   # only fmha_bwd_bf16.npz
    python tests/golden/make_golden.py backward256  # only fmha_bwd_h256_bf16.npz
"""
import os

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.uint16).numpy().copy()


def backward(H=64, seed=4321, shape=(1, 2, 140, 150), filename="fmha_bwd_bf16.npz"):
    """Attention gradients by autograd over plain fp32 attention: causal, and non-causal with a
    head-broadcast additive bias; ragged sizes.  Head size 64, and 256 (the head size of the two
    decoder-layer configurations) in a file of its own."""
    torch.manual_seed(seed)
    torch.set_num_threads(1)
    B, Nh, F, T = shape
    scale = H ** -0.5
    q, k, v = (torch.randn(B, Nh, S, H).bfloat16() for S in (F, T, T))
    do = torch.randn(B, Nh, F, H).bfloat16()
    bias = (torch.randn(B, 1, F, T) * 0.5).bfloat16()
    out = {"q": bits(q), "k": bits(k), "v": bits(v), "do": bits(do), "bias": bits(bias), "scale": np.float32(scale)}
    for name in ("causal", "bias"):
        qf, kf, vf = (t.float().requires_grad_() for t in (q, k, v))
        s = torch.einsum("bnfh,bnth->bnft", qf, kf) * scale
        if name == "causal":
            s = s.masked_fill(~torch.ones(F, T, dtype=torch.bool).tril(), float("-inf"))
        else:
            s = s + bias.float()
        o = torch.softmax(s, dim=-1) @ vf
        o.backward(do.float())
        out.update({f"o_{name}": o.detach().numpy(), f"lse_{name}": torch.logsumexp(s, dim=-1).detach().numpy(),
                    f"dq_{name}": qf.grad.numpy(), f"dk_{name}": kf.grad.numpy(), f"dv_{name}": vf.grad.numpy()})
    np.savez_compressed(os.path.join(HERE, filename), **out)


def backward256():
    backward(H=256, seed=8765, shape=(1, 2, 72, 90), filename="fmha_bwd_h256_bf16.npz")


def main():
    torch.manual_seed(1234)
    torch.set_num_threads(1)

    # ---- GEMM + bias + GELU(tanh), bf16, and + beta*C
    M, K, N = 96, 80, 72
    x = torch.randn(M, K).bfloat16()
    w = (torch.randn(K, N) * 0.1).bfloat16()
    b = (torch.randn(N) * 0.1).bfloat16()
    c = torch.randn(M, N).bfloat16()
    acc = x.float() @ w.float()
    out_gelu = torch.nn.functional.gelu(acc + b.float(), approximate="tanh").bfloat16()
    out_bias_res = (acc + b.float() + 0.5 * c.float()).bfloat16()
    out_relu = torch.relu(acc).bfloat16()
    np.savez_compressed(os.path.join(HERE, "gemm_bf16.npz"), x=bits(x), w=bits(w), b=bits(b), c=bits(c),
                        out_bias_gelu=bits(out_gelu), out_bias_beta=bits(out_bias_res), out_relu=bits(out_relu),
                        beta=np.float32(0.5))

    # ---- attention: causal, and non-causal with a head-broadcast additive bias; fp16 ragged
    B, Nh, F, T, H = 2, 3, 40, 56, 64
    q = torch.randn(B, Nh, F, H).bfloat16()
    k = torch.randn(B, Nh, T, H).bfloat16()
    v = torch.randn(B, Nh, T, H).bfloat16()
    bias = torch.randn(B, 1, F, T).bfloat16()
    scale = H ** -0.5
    sdpa = torch.nn.functional.scaled_dot_product_attention
    # top-left anchored causal mask (t <= f), as the reference's kernel defines it
    mask = torch.ones(F, T, dtype=torch.bool).tril()
    o_causal = sdpa(q.float(), k.float(), v.float(), attn_mask=mask, scale=scale)
    o_bias = sdpa(q.float(), k.float(), v.float(), attn_mask=bias.float(), scale=scale)
    s = torch.einsum("bnfh,bnth->bnft", q.float(), k.float()) * scale + bias.float()
    lse_bias = torch.logsumexp(s, dim=-1)
    np.savez_compressed(os.path.join(HERE, "fmha_bf16.npz"), q=bits(q), k=bits(k), v=bits(v), bias=bits(bias),
                        o_causal=o_causal.numpy(), o_bias=o_bias.numpy(), lse_bias=lse_bias.numpy(),
                        scale=np.float32(scale))

    B, Nh, F, T, H = 1, 2, 33, 77, 40
    q = torch.randn(B, Nh, F, H).half()
    k = torch.randn(B, Nh, T, H).half()
    v = torch.randn(B, Nh, T, H).half()
    o = sdpa(q.float(), k.float(), v.float(), scale=H ** -0.5)
    np.savez_compressed(os.path.join(HERE, "fmha_f16_ragged.npz"), q=bits(q), k=bits(k), v=bits(v), o=o.numpy(),
                        scale=np.float32(H ** -0.5))

    # ---- fp8: torch's casts as the independent quantiser; fp32 matmul of dequantised operands
    a = torch.randn(64, 96)
    bm = torch.randn(96, 48)
    out = {}
    for name, dt in (("e4m3", torch.float8_e4m3fn), ("e5m2", torch.float8_e5m2)):
        fmax = torch.finfo(dt).max
        sa = fmax / a.abs().max().item()
        sb = fmax / bm.abs().max().item()
        aq = (a * sa).clamp(-fmax, fmax).to(dt)
        bq = (bm * sb).clamp(-fmax, fmax).to(dt)
        ref = (aq.float() / sa) @ (bq.float() / sb)
        out.update({f"aq_{name}": aq.view(torch.uint8).numpy(), f"bq_{name}": bq.view(torch.uint8).numpy(),
                    f"sa_{name}": np.float64(sa), f"sb_{name}": np.float64(sb), f"ref_{name}": ref.numpy()})
    # a sweep of values for the cast itself, including ties, subnormals and overflow
    sweep = torch.cat([torch.linspace(-600, 600, 4001), torch.linspace(-1, 1, 4001) * 2 ** -6,
                       torch.tensor([0.0, -0.0, 448.0, 464.0, 480.0, 1e9, -1e9, 2 ** -9, 2 ** -10, 57344.0, 61440.0, 7e4])])
    out["sweep"] = sweep.numpy()
    out["sweep_e4m3"] = sweep.clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    out["sweep_e5m2"] = sweep.clamp(-57344, 57344).to(torch.float8_e5m2).view(torch.uint8).numpy()
    np.savez_compressed(os.path.join(HERE, "fp8.npz"), a=a.numpy(), b=bm.numpy(), **out)
    print("wrote", sorted(f for f in os.listdir(HERE) if f.endswith(".npz")))


if __name__ == "__main__":
    import sys
    if sys.argv[1:] == ["backward"]:
        backward()
    elif sys.argv[1:] == ["backward256"]:
        backward256()
    else:
        main()
        backward()
        backward256()
