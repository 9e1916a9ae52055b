#!/usr/bin/env python3
"""Tensor-parallel training step of a Llama-style decoder (RMSNorm, causal attention, SwiGLU) under the Megatron
placement: wq, wk, wv, w1, w3 cut by rows, wo and w2 by columns; forward and backward in one compiled program.
The counterpart of the reference's canonical example (examples/parallel.py:25-89), at its sizes by default."""
import torch

from common import arguments, execute, units_of


def main(argv=None):
    args = arguments(__doc__, argv)
    from mesh_b200.models.llama import Decoder, megatron
    torch.manual_seed(0)
    dim, heads, ffn, layers, batch, seq = (64, 4, 128, 2, 2, 16) if args.small else (2048, 16, 5632, 4, 2, 1024)
    model = Decoder(dim=dim, heads=heads, ffn=ffn, layers=layers).to(args.device)
    x = torch.randn(batch, seq, dim, device=args.device)
    return execute(model, (x,), lambda procs: megatron(procs, units_of(args)), args, loss=0)


if __name__ == "__main__":
    main()
