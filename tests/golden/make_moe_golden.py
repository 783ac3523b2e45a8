"""Generates tests/golden/moe_torch.npz: router, alignment, grouped-GEMM and combine vectors computed with
PyTorch's own operators (softmax, topk, stable argsort, bincount, cumsum, matmul, index_add_) on the CPU, an
implementation independent of the restatements under oracle/.  Run from the repository root:

    python tests/golden/make_moe_golden.py

Cases avoid exact ties in the router (torch.topk does not promise the lowest index on ties; the tie rule is
pinned by hand-written vectors instead): a case is redrawn until the k-th and (k+1)-th probabilities differ.
"""
import os

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def router_case(seed, T, E, k):
    g = torch.Generator().manual_seed(seed)
    while True:
        logits = torch.randn(T, E, generator=g, dtype=torch.float32)
        prob = torch.softmax(logits, dim=-1)
        top = torch.topk(prob, min(k + 1, E), dim=-1)
        gaps = top.values[:, :-1] - top.values[:, 1:]
        if E == k or float(gaps.min()) > 1e-6:
            break
    w = top.values[:, :k].contiguous()
    idx = top.indices[:, :k].to(torch.int32).contiguous()
    wn = w / w.sum(dim=-1, keepdim=True)
    return logits.numpy(), w.numpy(), wn.numpy(), idx.numpy()


def align_case(ids, E, block):
    """Stable sort of the flat slots by expert, every expert's run padded to a multiple of `block`."""
    T, k = ids.shape
    flat = torch.from_numpy(ids.reshape(-1).astype(np.int64))
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=E)
    padded = (counts + block - 1) // block * block
    starts = torch.cumsum(padded, 0) - padded
    max_padded = T * k + E * (block - 1)
    sorted_ids = torch.full((max_padded,), T * k, dtype=torch.int32)
    experts_ids = torch.zeros((max_padded // block,), dtype=torch.int32)
    src = 0
    for e in range(E):
        c = int(counts[e])
        sorted_ids[int(starts[e]) : int(starts[e]) + c] = order[src : src + c].to(torch.int32)
        experts_ids[int(starts[e]) // block : (int(starts[e]) + int(padded[e])) // block] = e
        src += c
    return sorted_ids.numpy(), experts_ids.numpy(), int(padded.sum())


def main():
    out = {}
    for name, (seed, T, E, k) in {"mixtral": (11, 256, 8, 2), "wide": (12, 33, 64, 6), "qwen": (13, 5, 128, 8),
                                  "all": (14, 7, 4, 4)}.items():
        lg, w, wn, idx = router_case(seed, T, E, k)
        out[f"router_{name}_logits"], out[f"router_{name}_w"] = lg, w
        out[f"router_{name}_wnorm"], out[f"router_{name}_idx"] = wn, idx
        for block in (4, 64):
            s, e, npp = align_case(idx, E, block)
            out[f"align_{name}_b{block}_sorted"], out[f"align_{name}_b{block}_experts"] = s, e
            out[f"align_{name}_b{block}_npp"] = np.array([npp], dtype=np.int32)

    # grouped GEMM by slot and the weighted combine, f64 in torch
    g = torch.Generator().manual_seed(21)
    T, H, N, E, k = 19, 64, 24, 6, 3
    A = torch.randn(T, H, generator=g, dtype=torch.float32).bfloat16().float()
    B = (torch.randn(E, N, H, generator=g, dtype=torch.float32) * 0.1).bfloat16().float()
    ids = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int32)
    w = torch.rand(T, k, generator=g, dtype=torch.float32) * 0.9 + 0.1
    slot_tok = torch.arange(T * k) // k
    C = torch.einsum("sh,snh->sn", A[slot_tok].double(), B[ids.reshape(-1).long()].double())
    Cw = C * w.reshape(-1, 1).double()
    y = torch.zeros(T, N, dtype=torch.float64).index_add_(0, slot_tok, Cw)
    out.update(gemm_A=A.numpy(), gemm_B=B.numpy(), gemm_ids=ids.numpy(), gemm_w=w.numpy(), gemm_C=C.numpy(),
               gemm_Cw=Cw.numpy(), gemm_y=y.numpy())
    np.savez_compressed(os.path.join(HERE, "moe_torch.npz"), **out)
    print("wrote moe_torch.npz:", len(out), "arrays")


if __name__ == "__main__":
    main()
