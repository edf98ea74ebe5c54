"""The Hugging Face patch layer (reference: cut_cross_entropy/transformers/patch.py, utils.py).

CPU tests cover the patching mechanics (no kernel runs without labels); the GPU tests compare a
patched tiny model with the unpatched one: same loss, same parameter gradients.
"""

from __future__ import annotations

import copy

import pytest
import torch

transformers = pytest.importorskip("transformers")


def _tiny(model_type: str):
    if model_type == "llama":
        from transformers import LlamaConfig, LlamaForCausalLM

        cfg = LlamaConfig(vocab_size=1003, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                          num_attention_heads=4, num_key_value_heads=2)  # fmt: skip
        return LlamaForCausalLM(cfg)
    if model_type == "gemma2":
        from transformers import Gemma2Config, Gemma2ForCausalLM

        cfg = Gemma2Config(vocab_size=1003, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                           num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                           final_logit_softcapping=30.0, sliding_window=16)  # fmt: skip
        return Gemma2ForCausalLM(cfg)
    if model_type == "qwen2":
        from transformers import Qwen2Config, Qwen2ForCausalLM

        cfg = Qwen2Config(vocab_size=1003, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                          num_attention_heads=4, num_key_value_heads=2)  # fmt: skip
        return Qwen2ForCausalLM(cfg)
    raise ValueError(model_type)


def test_patch_mechanics_on_cpu():
    from cut_cross_entropy.transformers import cce_patch
    from cut_cross_entropy.transformers.patch import cce_unpatch
    from cut_cross_entropy.transformers.utils import PatchOptions

    torch.manual_seed(0)
    model = _tiny("llama")
    ids = torch.randint(0, 1003, (2, 9))
    ref = model(input_ids=ids)
    assert cce_patch(model) is model
    out = model(input_ids=ids)  # no labels: the model's own forward
    assert torch.equal(out.logits, ref.logits)
    with pytest.raises(RuntimeError, match="no CPU path"):
        model(input_ids=ids, labels=ids)  # labels: the fused loss, which needs the GPU
    # train_only: in eval mode the original loss path runs, also with labels
    model = cce_patch(_tiny("llama"), train_only=True).eval()
    assert model(input_ids=ids, labels=ids).logits is not None

    with pytest.raises(RuntimeError, match="Unknown model type"):
        cce_patch("bert")
    with pytest.raises(ValueError, match="Unknown"):
        cce_patch("llama", impl="nope")
    with pytest.raises(NotImplementedError):
        cce_patch("llama", impl="torch_compile")

    # class-level patch by model type or config, and its undo
    from transformers.models.llama.modeling_llama import LlamaForCausalLM

    before = LlamaForCausalLM.forward
    assert cce_patch("llama") is None
    assert LlamaForCausalLM.forward is not before and getattr(LlamaForCausalLM.forward, "__cce_patched__", False)
    assert cce_patch(_tiny("llama").config, reduction="sum") is None
    cce_unpatch("llama")
    assert LlamaForCausalLM.forward is before

    o = PatchOptions("cce", "mean", "auto", False, False, True, True, train_only=True)
    assert not o.use_lce(None, True) and o.use_lce(ids, True) and not o.use_lce(ids, False)
    assert set(o.to_kwargs()) == {"impl", "reduction", "filter_eps", "accum_e_fp32", "accum_c_fp32",
                                  "filter_e_grad", "filter_c_grad"}  # fmt: skip


@pytest.mark.gpu
@pytest.mark.parametrize("model_type", ["llama", "gemma2", "qwen2"])
@pytest.mark.parametrize("num_items", [None, 37])
def test_patched_model_matches_unpatched(model_type, num_items):
    from cut_cross_entropy.transformers import cce_patch

    torch.manual_seed(1)
    base = _tiny(model_type).to("cuda", torch.bfloat16).train()
    patched = cce_patch(copy.deepcopy(base), impl="cce_exact")
    ids = torch.randint(0, 1003, (3, 40), device="cuda")
    labels = ids.clone()
    labels[:, :5] = -100
    kw = {} if num_items is None else {"num_items_in_batch": num_items}
    ref = base(input_ids=ids, labels=labels, **kw)
    out = patched(input_ids=ids, labels=labels, **kw)
    assert out.logits is None
    assert abs(out.loss.item() - ref.loss.item()) <= 5e-3 * abs(ref.loss.item()) + 1e-3
    ref.loss.backward()
    out.loss.backward()
    for (name, p_ref), (_, p_out) in zip(base.named_parameters(), patched.named_parameters()):
        if p_ref.grad is None:
            continue
        g_ref, g_out = p_ref.grad.float(), p_out.grad.float()
        scale = g_ref.abs().max().item() + 1e-6
        assert (g_ref - g_out).abs().max().item() <= 5e-2 * scale, name
        cos = torch.nn.functional.cosine_similarity(g_ref.flatten(), g_out.flatten(), dim=0).item()
        assert cos >= 0.99, (name, cos)
