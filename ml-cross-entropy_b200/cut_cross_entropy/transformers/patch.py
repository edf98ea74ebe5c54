"""``cce_patch``: switch a ``transformers`` causal LM to the fused linear-cross-entropy loss.

Same entry point and options as the reference (``cut_cross_entropy/transformers/patch.py:53-91``).
The reference carries a copy of each model's ``forward`` written against transformers 4.48; the
causal-LM forwards of transformers 5.x share one shape (decoder -> ``lm_head`` -> ``loss_function``),
so here ONE forward serves every supported architecture: it runs the decoder, hands the hidden
states and the ``lm_head`` weight to :func:`apply_lce` (with the logit soft-cap of the config, if
it has one: Gemma-2), and returns ``logits=None``.  Without labels, or in eval mode under
``train_only``, the model's original forward runs unchanged.
"""

from __future__ import annotations

import importlib
from types import MethodType

import torch

from ..cce_utils import LinearCrossEntropyImpl
from ..linear_cross_entropy import LCE_IMPL_DEFAULT
from .utils import PatchOptions, apply_lce

# model_type -> (module, class) of the causal-LM head it patches (the reference's five families)
SUPPORTED = {
    "llama": ("transformers.models.llama.modeling_llama", "LlamaForCausalLM"),
    "mistral": ("transformers.models.mistral.modeling_mistral", "MistralForCausalLM"),
    "qwen2": ("transformers.models.qwen2.modeling_qwen2", "Qwen2ForCausalLM"),
    "phi3": ("transformers.models.phi3.modeling_phi3", "Phi3ForCausalLM"),
    "gemma2": ("transformers.models.gemma2.modeling_gemma2", "Gemma2ForCausalLM"),
}


def _make_forward(original_forward, opts: PatchOptions):
    def cce_forward(
        self,
        input_ids=None,
        attention_mask=None,
        position_ids=None,
        past_key_values=None,
        inputs_embeds=None,
        labels=None,
        use_cache=None,
        logits_to_keep=0,
        **kwargs,
    ):
        if not opts.use_lce(labels, self.training):
            return original_forward(
                self, input_ids=input_ids, attention_mask=attention_mask, position_ids=position_ids,
                past_key_values=past_key_values, inputs_embeds=inputs_embeds, labels=labels, use_cache=use_cache,
                logits_to_keep=logits_to_keep, **kwargs,
            )  # fmt: skip
        from transformers.modeling_outputs import CausalLMOutputWithPast

        return_dict = kwargs.pop("return_dict", None)
        outputs = self.model(
            input_ids=input_ids, attention_mask=attention_mask, position_ids=position_ids,
            past_key_values=past_key_values, inputs_embeds=inputs_embeds, use_cache=use_cache, **kwargs,
        )  # fmt: skip
        hidden_states = outputs.last_hidden_state
        loss = apply_lce(
            hidden_states,
            self.lm_head.weight,
            labels,
            opts,
            bias=getattr(self.lm_head, "bias", None),
            softcap=getattr(self.config, "final_logit_softcapping", None),
            **kwargs,
        )
        out = CausalLMOutputWithPast(
            loss=loss,
            logits=None,
            past_key_values=outputs.past_key_values,
            hidden_states=outputs.hidden_states,
            attentions=outputs.attentions,
        )
        if return_dict is False:
            return out.to_tuple()
        return out

    cce_forward.__cce_patched__ = True
    return cce_forward


def cce_patch(
    model_type_or_model,
    impl: str | LinearCrossEntropyImpl = LCE_IMPL_DEFAULT,
    reduction: str = "mean",
    filter_eps: float | str | None = "auto",
    accum_e_fp32: bool = False,
    accum_c_fp32: bool = False,
    filter_e_grad: bool = True,
    filter_c_grad: bool = True,
    train_only: bool = False,
):
    """Patch a model instance (returned) or, given a model-type string or a config, the class (returns ``None``).

    Supported ``model_type``: llama, mistral, qwen2, phi3, gemma2.  ``impl="torch_compile"`` is not
    part of this backend and is refused.
    """
    import transformers

    if isinstance(impl, LinearCrossEntropyImpl):
        impl = impl.name.lower()
    if impl not in (v.name.lower() for v in LinearCrossEntropyImpl):
        raise ValueError(f"Unknown {impl=}")
    if impl == "torch_compile":
        raise NotImplementedError("torch_compile is not implemented by this backend.")

    if isinstance(model_type_or_model, transformers.PreTrainedModel):
        model_type = model_type_or_model.config.model_type
    elif isinstance(model_type_or_model, transformers.PretrainedConfig):
        model_type = model_type_or_model.model_type
    else:
        model_type = model_type_or_model
    if model_type not in SUPPORTED:
        raise RuntimeError(f"Unknown model type {model_type}")

    opts = PatchOptions(
        impl=impl,
        reduction=reduction,
        filter_eps=filter_eps,
        accum_e_fp32=accum_e_fp32,
        accum_c_fp32=accum_c_fp32,
        filter_e_grad=filter_e_grad,
        filter_c_grad=filter_c_grad,
        train_only=train_only,
    )
    module_name, class_name = SUPPORTED[model_type]
    cls = getattr(importlib.import_module(module_name), class_name)
    original = getattr(cls, "__cce_original_forward__", cls.forward)

    if isinstance(model_type_or_model, transformers.PreTrainedModel):
        model = model_type_or_model
        if not isinstance(model, cls):
            raise RuntimeError(f"Expected a {class_name} for model type {model_type}, got {type(model).__name__}")
        model.forward = MethodType(_make_forward(original, opts), model)
        return model

    if not hasattr(cls, "__cce_original_forward__"):
        cls.__cce_original_forward__ = cls.forward
    cls.forward = _make_forward(original, opts)
    return None


def cce_unpatch(model_type: str) -> None:
    """Undo a class-level patch (instances patched individually keep their own ``forward``)."""
    module_name, class_name = SUPPORTED[model_type]
    cls = getattr(importlib.import_module(module_name), class_name)
    if hasattr(cls, "__cce_original_forward__"):
        cls.forward = cls.__cce_original_forward__
        del cls.__cce_original_forward__
