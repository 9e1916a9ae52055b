"""Models of the ``transformers`` library (random weights, tiny configurations) through the compiler: a user's existing
model, unchanged, under a cut of the batch or of the sequence, against eager PyTorch.  Covers what such models bring that
the package's own models do not: attention called with a mask tensor, an output projection tied to the embedding
(one tensor under two parameter names), code after attention that relies on the fused operator's memory layout."""
import pytest
import torch
import torch.nn as nn

transformers = pytest.importorskip("transformers")

from mesh_b200.compiler import Program, archive, compile_module  # noqa: E402


class _Logits(nn.Module):
    def __init__(self, m):
        super().__init__()
        self.m = m

    def forward(self, ids):
        return self.m(input_ids=ids, use_cache=False).logits


class _Loss(nn.Module):
    def __init__(self, m):
        super().__init__()
        self.m = m

    def forward(self, ids):
        return self.m(input_ids=ids, labels=ids, use_cache=False).loss


def _llama(tie=False):
    cfg = transformers.LlamaConfig(vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                                   num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=64,
                                   tie_word_embeddings=tie)
    return transformers.LlamaForCausalLM(cfg)


def _gpt2():
    cfg = transformers.GPT2Config(vocab_size=128, n_embd=64, n_layer=2, n_head=4, n_positions=64, resid_pdrop=0.0,
                                  embd_pdrop=0.0, attn_pdrop=0.0)
    return transformers.GPT2LMHeadModel(cfg)          # the output projection is the embedding


def _place(x, dim, names):
    def place(node):
        val = node.meta.get("val")
        mine = node.op == "placeholder" and not node.name.startswith(("p_", "b_", "c_")) and getattr(val, "shape", None) == x.shape
        return (dim, names, None) if mine else None
    return place


@pytest.mark.parametrize("make", [_llama, _gpt2])
@pytest.mark.parametrize("dim", [0, 1])
def test_inference_logits_under_batch_and_sequence_cuts(make, dim):
    torch.manual_seed(0)
    model = make()
    model.config._attn_implementation = "sdpa"
    model = _Logits(model).eval()
    ids = torch.randint(0, 128, (4, 16))
    procs = {f"p{i}": (0, "cpu") for i in range(2)}
    sch = compile_module(model, (ids,), procs, _place(ids, dim, tuple(procs)), strict=False)
    prog = Program(sch)
    got, ref = prog(ids), model(ids)
    assert (got - ref).abs().max() <= 1e-5 * ref.abs().max()
    assert sch.structure["gathering_fallbacks"] == 0       # attention with its mask tensor keeps the cut
    # tokens cut: every layer's attention is a ring step that reads its mask by rows held and columns of the block at hand
    assert prog.fusion["ring_attention"] == (2 if dim == 1 else 0)


@pytest.mark.parametrize("make,dim", [(_llama, 0), (_llama, 1), (_gpt2, 0), (_gpt2, 1)])
def test_training_step_matches_eager_and_tied_names_carry_the_summed_gradient(make, dim, tmp_path):
    torch.manual_seed(0)
    model = make()
    model.config._attn_implementation = "sdpa"
    model = _Loss(model).train()
    ids = torch.randint(0, 128, (4, 16))
    procs = {f"p{i}": (0, "cpu") for i in range(2)}
    sch = compile_module(model, (ids,), procs, _place(ids, dim, tuple(procs)), strict=False, loss=0)
    tied = make is _gpt2
    assert bool(sch.exported.tied) == tied
    shared = dict(model.named_parameters(remove_duplicate=False))
    if tied:                                               # the capture's stand-ins are gone: one tensor again
        assert shared["m.lm_head.weight"] is shared["m.transformer.wte.weight"]
        archive.save(tmp_path, sch)
        sch = archive.load(tmp_path)
        assert sch.exported.tied == {"m.lm_head.weight": "m.transformer.wte.weight"}
    res = Program(sch)(ids)
    ref = model(ids)
    ref.backward()
    assert abs(float(res.outputs.detach()) - float(ref.detach())) <= 1e-5 * abs(float(ref.detach()))
    scale = max(float(p.grad.abs().max()) for p in model.parameters())
    for name, g in res.parameters.items():
        r = shared[name].grad
        assert g.shape == r.shape and (g - r).abs().max() <= 2e-5 * scale, name
    if tied:
        assert torch.equal(res.parameters["m.lm_head.weight"], res.parameters["m.transformer.wte.weight"])


@pytest.mark.parametrize("train", [False, True])
def test_megatron_placement_by_parameter_names_costs_the_textbook_all_reduces(train):
    """``placements.tensor_parallel`` with the Llama family's names: two all-reduces per layer forward, two more
    backward, nothing gathered; the partial input gradient of a column-parallel layer, read by both the norm's input
    gradient and its weight gradient, is summed once."""
    from mesh_b200.compiler import placements
    torch.manual_seed(0)
    model = _llama()
    model.config._attn_implementation = "sdpa"
    model = (_Loss(model) if train else _Logits(model)).train(train)
    ids = torch.randint(0, 128, (4, 16))
    procs = {f"p{i}": (0, "cpu") for i in range(2)}
    place = placements.tensor_parallel(tuple(procs), **placements.LLAMA)
    sch = compile_module(model, (ids,), procs, place, strict=False, **({"loss": 0} if train else {}))
    layers = 2
    assert sch.structure["by_verb"] == {"all_reduce": (4 if train else 2) * layers}
    assert sch.structure["gathering_fallbacks"] == 0
    res = Program(sch)(ids)
    ref = model(ids)
    if not train:
        assert (res - ref).abs().max() <= 1e-5 * ref.abs().max()
        return
    ref.backward()
    assert abs(float(res.outputs.detach()) - float(ref.detach())) <= 1e-5 * abs(float(ref.detach()))
    scale = max(float(p.grad.abs().max()) for p in model.parameters())
    for name, g in res.parameters.items():
        r = dict(model.named_parameters())[name].grad
        if g.shape != r.shape:                               # a cut weight: this processor's block
            r = r[tuple(slice(0, n) for n in g.shape)]
        assert (g - r).abs().max() <= 2e-5 * scale, name


def test_row_parallel_layers_with_a_bias_keep_their_partial_sums():
    """BERT's projections carry biases.  Megatron placement by names: the row-parallel layers add their bias through the
    first processor only, so their results stay partial sums - two all-reduces per layer and nothing gathered."""
    from mesh_b200.compiler import placements
    torch.manual_seed(0)
    cfg = transformers.BertConfig(vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                                  num_attention_heads=4, max_position_embeddings=64, hidden_dropout_prob=0.0,
                                  attention_probs_dropout_prob=0.0)
    bert = transformers.BertModel(cfg)
    bert.config._attn_implementation = "sdpa"

    class Hidden(nn.Module):
        def __init__(self, m):
            super().__init__()
            self.m = m

        def forward(self, ids):
            return self.m(input_ids=ids).last_hidden_state
    model = Hidden(bert).eval()
    ids = torch.randint(0, 128, (4, 16))
    procs = {f"p{i}": (0, "cpu") for i in range(2)}
    place = placements.tensor_parallel(tuple(procs), column=("query", "key", "value", "intermediate_dense"),
                                       row=("attention_output_dense", r"layer_\d+_output_dense"))
    sch = compile_module(model, (ids,), procs, place, strict=False)
    assert sch.structure["by_verb"] == {"all_reduce": 4} and sch.structure["gathering_fallbacks"] == 0
    once = [st for st in sch.plan.steps if "once" in st.meta]
    assert len(once) == 4                                     # the four row-parallel layers
    got, ref = Program(sch)(ids), model(ids)
    assert (got - ref).abs().max() <= 1e-5 * ref.abs().max()


def _vit():
    cfg = transformers.ViTConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, image_size=32,
                                 patch_size=8, num_labels=5, hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)
    return (transformers.ViTForImageClassification(cfg), (torch.randn(4, 3, 32, 32), torch.randint(0, 5, (4,))),
            lambda m, x, y: m(pixel_values=x, labels=y).loss)


def _resnet():
    cfg = transformers.ResNetConfig(num_channels=3, embedding_size=8, hidden_sizes=[8, 16], depths=[1, 1], layer_type="basic", num_labels=5)
    return (transformers.ResNetForImageClassification(cfg), (torch.randn(4, 3, 32, 32), torch.randint(0, 5, (4,))),
            lambda m, x, y: m(pixel_values=x, labels=y).loss)


def _t5():
    cfg = transformers.T5Config(vocab_size=128, d_model=64, d_kv=16, d_ff=128, num_layers=2, num_heads=4, dropout_rate=0.0,
                                decoder_start_token_id=0, pad_token_id=0)
    return (transformers.T5ForConditionalGeneration(cfg), (torch.randint(0, 128, (4, 12)), torch.randint(0, 128, (4, 8))),
            lambda m, x, y: m(input_ids=x, labels=y).loss)


class _Call(nn.Module):
    def __init__(self, m, f):
        super().__init__()
        self.m, self.f = m, f

    def forward(self, *a):
        return self.f(self.m, *a)


@pytest.mark.parametrize("family", [_vit, _resnet, _t5])
def test_other_families_train_under_a_batch_cut(family):
    """A vision transformer (patch-embedding convolution), a residual network (training-mode batch norm: captured again
    with its statistics as sums) and an encoder-decoder with one table under four names, data-parallel on two
    processors: eager's loss and gradients."""
    torch.manual_seed(0)
    base, inputs, call = family()
    try:
        base.config._attn_implementation = "sdpa"
    except Exception:
        pass
    model = _Call(base, call).train()
    procs = {f"p{i}": (0, "cpu") for i in range(2)}
    names = tuple(procs)

    def place(node):
        val = node.meta.get("val")
        user = node.op == "placeholder" and not node.name.startswith(("p_", "b_", "c_"))
        return (0, names, None) if user and getattr(val, "ndim", 0) >= 1 and val.shape[0] == 4 else None
    sch = compile_module(model, inputs, procs, place, strict=False, loss=0)
    res = Program(sch)(*inputs)
    ref = model(*inputs)
    ref.backward()
    assert abs(float(res.outputs.detach()) - float(ref.detach())) <= 1e-5 * max(1.0, abs(float(ref.detach())))
    scale = max(float(p.grad.abs().max()) for p in model.parameters() if p.grad is not None)
    shared = dict(model.named_parameters(remove_duplicate=False))
    checked = 0
    for name, g in res.parameters.items():
        r = shared[name].grad
        if r is None or g is None:
            continue
        assert g.shape == r.shape and (g - r).abs().max() <= 3e-5 * scale, name
        checked += 1
    assert checked >= 10
