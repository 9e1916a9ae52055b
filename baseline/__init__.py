"""Plain PyTorch + torch.distributed (NCCL) + cuBLAS restatements of the reference's example models.

These are the "thing to beat": the reference itself targets Apple Silicon and cannot run on this
hardware, so its torch-level TP / EP / CP / PP examples are restated with stock library calls.
None of mesh_b200's kernels or runtime is used here.
"""
