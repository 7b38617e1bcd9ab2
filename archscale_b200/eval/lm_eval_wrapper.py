"""lm-evaluation-harness adapter: registers the model type ``ArchScale`` (`eval.py:144-234`).

    lm_eval --model ArchScale --model_args pretrained=<ckpt.pth>,config=<registry name> --tasks ... \
        --include_path <dir of this file>      # or: python -m archscale_b200.eval.lm_eval_wrapper <lm_eval args>

The harness (``lm_eval``) is an optional dependency; importing this module without it raises ImportError with
that message, nothing else in the package depends on it.
"""
from __future__ import annotations

import torch

try:
    from lm_eval.api.registry import register_model
    from lm_eval.models.huggingface import HFLM
    from lm_eval.models.utils import stop_sequences_criteria
except ImportError as e:  # pragma: no cover - optional dependency
    raise ImportError("archscale_b200.eval.lm_eval_wrapper needs the `lm_eval` package (lm-evaluation-harness)") from e

from archscale_b200.eval.common import load_model


@register_model("ArchScale")
class ArchScaleEvalWrapper(HFLM):
    def __init__(self, pretrained=None, config=None, max_length=4096, batch_size=1, device="cuda", dtype=torch.bfloat16,
                 backend="causal", tokenizer="Orkhan/llama-2-7b-absa", **kwargs):
        self._archscale_config = config
        super().__init__(pretrained=pretrained, max_length=max_length, batch_size=batch_size, device=device, dtype=dtype,
                         backend=backend, tokenizer=tokenizer, **kwargs)

    def _get_config(self, *args, **kwargs) -> None:
        self._config = None

    def _create_model(self, pretrained, dtype=torch.bfloat16, **kwargs) -> None:
        device = self.accelerator.device if hasattr(self, "accelerator") else str(self.device)
        self._model = load_model(pretrained, self._archscale_config, device, dtype)

    def _model_call(self, inps, attn_mask=None, labels=None):
        with torch.no_grad():
            return self.model(inps, attention_mask=attn_mask).logits

    def _model_generate(self, context, max_length, stop, **generation_kwargs):
        generation_kwargs["temperature"] = generation_kwargs.get("temperature", 0.0)
        do_sample = generation_kwargs.get("do_sample")
        if generation_kwargs["temperature"] == 0.0 and do_sample is None:
            generation_kwargs["do_sample"] = do_sample = False
        if do_sample is False and generation_kwargs["temperature"] == 0.0:
            generation_kwargs.pop("temperature")
        criteria = stop_sequences_criteria(self.tokenizer, stop, context.shape[1], context.shape[0])
        return self.model.generate(input_ids=context, max_length=max_length, stopping_criteria=criteria,
                                   pad_token_id=self.tokenizer.pad_token_id, return_dict_in_generate=False,
                                   **generation_kwargs)


if __name__ == "__main__":  # pragma: no cover
    from lm_eval.__main__ import cli_evaluate
    cli_evaluate()
