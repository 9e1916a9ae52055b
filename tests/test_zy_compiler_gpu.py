"""Compiled programs on GPUs: the threaded interpreter on one device, and one process per GPU with fused pairs."""
import pytest
import torch
import torch.distributed as dist

pytestmark = pytest.mark.gpu


def _procs(n):
    return {f"p{i}": (0, f"cuda:{i}") for i in range(n)}


def test_threaded_program_on_one_gpu_matches_eager():
    from mesh_b200.compiler import Program, compile_module
    from mesh_b200.models.llama import Decoder, megatron
    torch.manual_seed(0)
    m = Decoder(dim=64, heads=4, ffn=128, layers=2)
    x = torch.randn(2, 16, 64)
    procs = _procs(2)
    out = Program(compile_module(m.eval(), (x,), procs, megatron(procs)), device="cuda", threads=True)(x)
    assert out.is_cuda and torch.allclose(out.cpu(), m(x), atol=1e-4)


def test_compiled_decoder_runs_on_this_packages_kernels():
    """One processor, bf16: every product, the attention and the norms of a compiled decoder run on the tcgen05 GEMM,
    the flash kernel and the RMSNorm kernel (no cuBLAS / SDPA step left), and the result matches fp32 eager."""
    from mesh_b200.compiler import Program, compile_module
    from mesh_b200.models.llama import Block
    from mesh_b200.utils.status import check_status
    torch.manual_seed(0)
    blocks = torch.nn.Sequential(Block(512, 4, 1024), Block(512, 4, 1024)).eval()
    x = torch.randn(2, 256, 512)
    ref = blocks(x)
    procs = {"p0": (0, "cuda:0")}
    sch = compile_module(blocks.bfloat16(), (x.bfloat16(),), procs, lambda node: None)
    prog = Program(sch, device="cuda", threads=True)
    out = prog(x.bfloat16())
    check_status()
    st = prog.structure()
    assert st["fused"]["rms_norm"] == 4, st
    assert st["kernels"]["eager"] == 0 and st["kernels"]["own"] == 2 * (7 + 1 + 2), st      # 7 products, attention, 2 norms
    err = (out.float().cpu() - ref).square().mean().sqrt() / ref.square().mean().sqrt()
    assert err < 2e-2, float(err)


def test_prepared_program_starts_as_cuda_graphs():
    """One processor on a GPU: every execution of the prepared program is one CUDA-graph launch on one of `copies`
    sets of storage; results match eager for every execution, also with two executions in flight."""
    from mesh_b200.compiler import compile_module, prepare
    from mesh_b200.models.llama import Block
    from mesh_b200.utils.status import check_status
    torch.manual_seed(0)
    blocks = torch.nn.Sequential(Block(512, 4, 1024)).eval()
    x = torch.randn(2, 256, 512)
    sch = compile_module(blocks.bfloat16(), (x.bfloat16(),), {"p0": (0, "cuda:0")}, lambda node: None)
    from mesh_b200.compiler import Program
    pr = prepare(sch, (x.bfloat16(),), copies=2, program=Program(sch, device="cuda", threads=True))
    assert pr.graphs
    refs = []
    for step in range(5):
        xi = (x * (0.5 + 0.25 * step)).bfloat16()
        pr.inputs()[0].copy_(xi)
        b = pr.start()
        out = pr.result(b).float().cpu()
        ref = blocks.float()(xi.float()) if step == 0 else blocks(xi.float())
        err = (out - ref).square().mean().sqrt() / ref.square().mean().sqrt()
        assert err < 2e-2, (step, float(err))
    check_status()
    pr.retire()


def _rank(rank, world, rdv):
    import mesh_b200.distributed.context as context
    from mesh_b200.compiler import Program, compile_module
    from mesh_b200.config import MeshConfig, set_config
    from mesh_b200.distributed.context import MeshContext
    from mesh_b200.models.llama import Decoder, megatron
    from mesh_b200.utils.status import check_status
    torch.cuda.set_device(rank)
    set_config(MeshConfig.from_env(heap_bytes=1 << 30))
    ctx = MeshContext(rank, world, torch.device("cuda", rank), rdv, dist.group.WORLD)
    context._ctx = ctx                                    # what init() does: the executor finds the heap through it
    torch.manual_seed(1)
    m = Decoder(dim=512, heads=4, ffn=1024, layers=2).eval()
    x = torch.randn(1, 128 * world, 512)
    procs = _procs(world)
    names = tuple(procs)
    tp = megatron(procs)

    def placement(node):
        if node.op == "placeholder" and node.name == "x":
            return (1, names, None)                       # tokens cut too: all-gather -> mm, mm -> reduce-scatter pairs
        return tp(node)
    ref = m(x)
    mb = m.bfloat16()
    sch = compile_module(mb, (x.bfloat16(),), procs, placement)
    prog = Program(sch)
    assert not prog.threads and prog.fusion["ag_mm"] >= 2 and prog.fusion["mm_rs"] >= 2, prog.fusion
    out = prog(x.bfloat16())
    torch.cuda.synchronize()
    check_status()
    st = prog.structure()
    assert st["kernels"]["eager"] == 0 and st["kernels"]["own"] > 0, st      # no cuBLAS / SDPA step in the compiled layer
    if out is not None:
        err = (out.float().cpu() - ref).abs().max() / ref.abs().max()
        assert err < 5e-2, float(err)
    rdv.barrier("compiled-done")
    ctx.heap.close()


def test_one_process_per_gpu_runs_fused_pairs():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from mesh_b200.utils.launch import spawn_ranks
    spawn_ranks(_rank, 2, use_cuda=True, timeout=300.0, init_pg="nccl")
