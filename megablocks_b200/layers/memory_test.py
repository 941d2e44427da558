"""Peak-memory check of one dMoE layer (reference: megablocks/layers/memory_test.py:1-102).

Runs forward + backward of a bf16 dMoE on ``(batch, seq, hidden, ffn, experts, top_k)`` =
(8, 2048, 4096, 4096, 32, 4) by default, prints the peak allocated / reserved bytes,
the bytes of weights and of everything else (activations, workspaces), and a census of
the live CUDA tensors.  ``--memory-optimized`` switches activation recompute on.

    python -m megablocks_b200.layers.memory_test [--memory-optimized] [--impl grouped|sparse]
"""

import argparse
import gc

import torch

import megablocks_b200 as mb


def live_tensor_census(limit: int = 20):
    seen, rows = set(), []
    for obj in gc.get_objects():
        try:
            if torch.is_tensor(obj) and obj.is_cuda and obj.data_ptr() not in seen:
                seen.add(obj.data_ptr())
                rows.append((obj.numel() * obj.element_size(), tuple(obj.shape), str(obj.dtype)))
        except Exception:
            continue
    rows.sort(reverse=True)
    return rows[:limit]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--shape', type=int, nargs=6, default=[8, 2048, 4096, 4096, 32, 4],
                    metavar=('BS', 'SL', 'HS', 'FFN', 'E', 'K'))
    ap.add_argument('--impl', choices=['grouped', 'sparse'], default='grouped')
    ap.add_argument('--memory-optimized', action='store_true')
    args = ap.parse_args()
    bs, sl, hs, ffn, ne, top_k = args.shape
    device = torch.device('cuda', 0)
    margs = mb.Arguments(hidden_size=hs, ffn_hidden_size=ffn, moe_num_experts=ne, moe_top_k=top_k, fp16=False,
                         bf16=True, device=device, mlp_impl=args.impl, memory_optimized_mlp=args.memory_optimized)
    layer = mb.dMoE(margs)
    weight_bytes = sum(p.numel() * p.element_size() for p in layer.parameters())
    x = torch.randn(sl, bs, hs, device=device, dtype=torch.bfloat16).requires_grad_(True)
    torch.cuda.reset_peak_memory_stats()
    out, _ = layer(x)
    out.sum().backward()
    torch.cuda.synchronize()
    peak = torch.cuda.max_memory_allocated()
    print(f'shape (bs, sl, hs, ffn, experts, top_k) = {tuple(args.shape)}  impl={args.impl} '
          f'memory_optimized={args.memory_optimized}')
    print(f'max memory allocated = {peak / 2**30:.3f} GiB, reserved = {torch.cuda.max_memory_reserved() / 2**30:.3f} GiB')
    print(f'weights = {weight_bytes / 2**30:.3f} GiB, gradients = {weight_bytes / 2**30:.3f} GiB, '
          f'activations and workspaces = {(peak - 2 * weight_bytes) / 2**30:.3f} GiB')
    print('largest live tensors:')
    for nbytes, shape, dtype in live_tensor_census():
        print(f'  {nbytes / 2**20:10.1f} MiB  {shape}  {dtype}')


if __name__ == '__main__':
    main()
