"""Benchmarks of the named workloads, each with this package's path (``--impl mesh``) and a stock
PyTorch + NCCL + cuBLAS arm (``--impl baseline``).  Run one rank per GPU with ``python -m torch.distributed.run``;
every script prints one JSON line on rank 0, device-timed with CUDA events, max over ranks."""
