"""The placement library (``compiler/placements.py``): placements stated by name patterns, on the package's decoder."""
import torch
import torch.nn as nn

from mesh_b200.compiler import Program, compile_module, placements
from mesh_b200.models.llama import Decoder


def _procs(n):
    return {f"p{i}": (0, "cpu") for i in range(n)}


def _eager(m, *a):
    for p in m.parameters():
        p.grad = None
    loss = m(*a)
    loss.backward()
    return loss.detach(), {k: p.grad.clone() for k, p in m.named_parameters()}


def _close(res, loss, grads, tol=2e-5):
    assert abs(float(res.outputs.detach()) - float(loss)) <= tol * max(1.0, abs(float(loss)))
    scale = max(float(g.abs().max()) for g in grads.values())
    for k, g in res.parameters.items():
        r = grads[k]
        if g.shape != r.shape:
            r = r[tuple(slice(0, n) for n in g.shape)]
        assert (g - r).abs().max() <= tol * scale, k


def test_tensor_parallel_by_names_matches_the_models_own_placement():
    torch.manual_seed(0)
    m = Decoder(dim=48, heads=4, ffn=96, layers=2)
    x = torch.randn(2, 12, 48)
    procs = _procs(2)
    place = placements.tensor_parallel(tuple(procs), column=("wq", "wk", "wv", "w1", "w3"), row=("wo", "w2"))
    sch = compile_module(m, (x,), procs, place, loss=0)
    assert set(sch.structure["by_verb"]) == {"all_reduce"} and sch.structure["fallbacks"] == 0
    cut = [k for k, v in sch.plan.input_specs.items() if any(s.kind == "S" for s in v)]
    assert len(cut) == 2 * 7                                   # seven projections per layer, nothing else
    _close(Program(sch)(x), *_eager(m, x))


def test_patterns_match_whole_path_components_only():
    match = placements._matcher(("q_proj", r"layers_[0-3]"))
    assert match("p_model_layers_0_self_attn_q_proj_weight") and match("p_model_layers_3_mlp_up_weight")
    assert not match("p_model_xq_proj_weight") and not match("p_model_layers_12_mlp_up_weight")


def test_pipeline_by_module_paths_and_data_parallel_combined():
    """Layers 0 and 1 on the first processor, 2 and 3 on the second: activations cross once forward and once backward;
    every parameter's gradient is produced where the parameter lives."""
    torch.manual_seed(1)
    m = Decoder(dim=32, heads=2, ffn=64, layers=4)
    x = torch.randn(2, 8, 32)
    procs = _procs(2)
    place = placements.pipeline({r"blocks\.[01]\.": "p0", r"blocks\.[23]\.": "p1"})
    sch = compile_module(m, (x,), procs, place, loss=0)
    sends = sch.structure["by_verb"].get("send_recv", 0)
    assert 2 <= sends <= 4 and set(sch.structure["by_verb"]) <= {"send_recv", "broadcast"}, sch.structure["by_verb"]
    _close(Program(sch)(x), *_eager(m, x))


class _Tagger(nn.Module):
    def __init__(self):
        super().__init__()
        self.embed = nn.Embedding(64, 16)
        self.proj = nn.Linear(16, 32)
        self.out = nn.Linear(32, 8)

    def forward(self, ids, labels):
        h = torch.relu(self.proj(self.embed(ids)))
        return nn.functional.cross_entropy(self.out(h).flatten(0, 1), labels.flatten())


def test_vocabulary_parallel_embedding_with_column_and_row_layers_and_cut_inputs():
    torch.manual_seed(2)
    m = _Tagger()
    ids, labels = torch.randint(0, 64, (4, 6)), torch.randint(0, 8, (4, 6))
    procs = _procs(2)
    names = tuple(procs)
    tp = placements.tensor_parallel(names, column=("proj",), row=("out",), vocabulary=("embed",))
    sch = compile_module(m, (ids, labels), procs, tp, loss=0)
    assert sch.plan.input_specs["p_embed_weight"][0].dim == 0 and sch.plan.input_specs["p_proj_bias"][0].kind == "S"
    _close(Program(sch)(ids, labels), *_eager(m, ids, labels))
    # the same model with every input cut along the batch instead: parameters whole, gradients all-reduced
    dp = placements.combine(placements.data_parallel(names, inputs=("ids", "labels")), lambda node: None)
    sch = compile_module(m, (ids, labels), procs, dp, loss=0)
    assert sch.structure["by_verb"].get("all_reduce", 0) >= len(list(m.parameters()))
    _close(Program(sch)(ids, labels), *_eager(m, ids, labels))


def test_training_graphs_keep_their_submodule_paths():
    """The joint forward+backward trace drops the nodes' submodule paths; the capture puts them back: nearly every
    operator of a training plan knows the model part it belongs to (what share solvers and pipelines go by), and the
    backward operators of a layer carry that layer's path."""
    from mesh_b200.compiler import shares
    torch.manual_seed(3)
    m = Decoder(dim=32, heads=2, ffn=64, layers=2)
    x = torch.randn(2, 8, 32)
    sch = compile_module(m, (x,), _procs(2), placements.data_parallel(("p0", "p1")), loss=0)
    calls = [n for n in sch.exported.graph_module.graph.nodes if n.op == "call_function"]
    with_path = [n for n in calls if n.meta.get("nn_module_stack")]
    assert len(with_path) >= 0.95 * len(calls)
    backward_of_w2 = [n for n in calls if "blocks.1.w2" in [q for q, _ in (n.meta.get("nn_module_stack") or {}).values()]]
    assert len(backward_of_w2) >= 4                       # the forward product, its two backward products, their views
    parts = {st.meta.get("module") for st in sch.plan.steps if st.op == "call"}
    assert {"blocks.0.w1", "blocks.1.wo", "blocks.1.attention_norm"} <= parts
    staged = shares.stages(sch)
    assert staged is not None


def test_pipeline_by_context_by_tensor_grid_compiles_and_trains():
    """A 2 x 2 x 2 grid with roles (pipeline stage, context, tensor): layers 0-1 on stage 0 and 2-3 on stage 1, tokens
    cut over the context axis, Megatron cuts over the tensor axis - one compiled training step on eight processors.
    Activations cross the stages once forward; nothing is gathered for want of a rule; loss and gradients are eager's."""
    torch.manual_seed(4)
    m = Decoder(dim=32, heads=4, ffn=64, layers=4)
    x = torch.randn(2, 8, 32)
    procs = _procs(8)
    place = placements.grid(("pp", "cp", "tp"), stages={r"blocks\.[01]\.": 0, r"blocks\.[23]\.": 1}, stage_axis="pp",
                            column=("wq", "wk", "wv", "w1", "w3"), row=("wo", "w2"), tensor_axis="tp",
                            inputs={"x": {"cp": 1}})
    sch = compile_module(m, (x,), procs, place, loss=0, mesh=(2, 2, 2))
    verbs = sch.structure["by_verb"]
    assert sch.structure["gathering_fallbacks"] == 0 and 2 <= verbs["send_recv"] <= 6 and verbs["all_reduce"] > 0
    specs = sch.plan.input_specs
    assert [s.kind for s in specs["p_blocks_0_wq_weight"]] == ["O", "R", "S"] and specs["p_blocks_0_wq_weight"][0].owner == 0
    assert specs["p_blocks_3_w2_weight"][0].owner == 1 and specs["p_blocks_3_w2_weight"][2].dim == 1
    assert [s.kind for s in specs["x"]] == ["O", "S", "R"]
    _close(Program(sch)(x), *_eager(m, x))
    # the same roles for inference: one crossing, attention's keys and values travel around the context axis
    m.eval()

    class Body(nn.Module):
        def __init__(self, d):
            super().__init__()
            self.blocks = d.blocks

        def forward(self, x):
            for b in self.blocks:
                x = b(x)
            return x
    body = Body(m).eval()
    sch = compile_module(body, (x,), procs, place, mesh=(2, 2, 2))
    prog = Program(sch)
    assert prog.fusion["ring_attention"] == 4 and sch.structure["by_verb"]["send_recv"] == 1
    ref = body(x)
    assert (prog(x) - ref).abs().max() <= 1e-5 * ref.abs().max()


def _grid_rank(rank, world, rdv):
    torch.manual_seed(5)
    m = Decoder(dim=32, heads=4, ffn=64, layers=2)
    x = torch.randn(2, 8, 32)
    procs = _procs(world)
    place = placements.grid(("pp", "cp", "tp"), stages={r"blocks\.0\.": 0, r"blocks\.1\.": 1}, stage_axis="pp",
                            column=("wq", "wk", "wv", "w1", "w3"), row=("wo", "w2"), tensor_axis="tp", inputs={"x": {"cp": 1}})
    sch = compile_module(m, (x,), procs, place, loss=0, mesh=(2, 2, 2))
    prog = Program(sch)
    assert not prog.threads
    res = prog(x)                                         # one process per processor: stages exchange point to point
    loss, grads = _eager(m, x)
    if res is not None and res.outputs is not None:
        assert abs(float(res.outputs.detach()) - float(loss)) <= 2e-5 * max(1.0, abs(float(loss)))
    if res is not None:
        scale = max(float(g.abs().max()) for g in grads.values())
        for k, g in res.parameters.items():
            if g is None:                                 # a parameter of the other stage
                continue
            r = grads[k]
            if g.shape != r.shape:
                continue                                  # a cut weight: checked by the threaded test above
            assert (g - r).abs().max() <= 2e-5 * scale, k


def test_grid_program_between_processes():
    from mesh_b200.utils.launch import spawn_ranks
    spawn_ranks(_grid_rank, 8, init_pg="gloo")
