"""``SharePrefill(...)(model)``: patch a Hugging Face decoder-only model in place.

Mirrors shareprefill_patch.py:31-169 of opas-lab/SharePrefill (Apache-2.0; the argument list, the
side effects and the error messages of that file are this boundary's contract): registers the attention function under the name
``"shareprefill"`` in the modeling module's ``ALL_ATTENTION_FUNCTIONS``, sets
``config._attn_implementation``, installs ``_init_attention_sharing`` /
``reset_attention_sharing`` on the model class, copies the knobs onto ``model.config`` at
every reset, points every attention module at the shared state object and wraps
``model.forward`` so that the state is reset before each call.

The reference additionally swaps ``model.model.forward`` for its own decoder loop
(model_patch.py:41-170) to avoid building a 4-D causal mask under transformers 4.51; newer
transformers build no mask for a custom attention name, and that loop does not run on them,
so the decoder forward is left untouched here.
"""
from __future__ import annotations

import functools
import importlib
import logging

from . import native
from .attention import shareprefill_attention_forward
from .configuration import SharePrefillConfig
from .sharing_state import AttentionSharing

LOGGER = logging.getLogger(__name__)


class SharePrefill:
    def __init__(
        self,
        attn_type: str = "shareprefill",
        model_name: str = None,
        sharing_lookup_path: str = None,
        pattern_threshold: float = 0.9,
        similarity_threshold: float = 0.5,
        fallback_threshold: float = 0.9,
        queryaware_threshold: float = 0.1,
        block_size: int = 128,
        min_budget: int = 1024,
        max_budget: int = None,
        **kwargs,
    ):
        self.config = SharePrefillConfig(
            attn_type=attn_type, model_name=model_name, sharing_lookup_path=sharing_lookup_path,
            pattern_threshold=pattern_threshold, similarity_threshold=similarity_threshold,
            fallback_threshold=fallback_threshold, queryaware_threshold=queryaware_threshold,
            block_size=block_size, min_budget=min_budget, max_budget=max_budget, **kwargs)

    def __call__(self, model):
        return self.patch_model(model)

    def patch_model(self, model):
        if self.config.attn_type in self.config.SUPPORTED_ATTENTION_TYPES:
            return shareprefill_patch(model, self.config)
        raise ValueError(f"The attention type {self.config.attn_type} is not supported.")


def shareprefill_patch(model, config: SharePrefillConfig):
    try:
        Attention = model.model.layers[0].self_attn.__class__
    except AttributeError as exc:
        raise TypeError("SharePrefill expects a decoder-only architecture exposing "
                        "`model.model.layers[*].self_attn`.") from exc

    attention_module = importlib.import_module(Attention.__module__)
    attention_functions = getattr(attention_module, "ALL_ATTENTION_FUNCTIONS", None)
    if attention_functions is None:
        raise TypeError("Expected the attention module to define ALL_ATTENTION_FUNCTIONS for integration.")
    attention_functions["shareprefill"] = shareprefill_attention_forward
    model.config._attn_implementation = "shareprefill"

    def _init_attention_sharing(self):
        self.attention_sharing = AttentionSharing(config.sharing_lookup_path)
        return self.attention_sharing

    def reset_attention_sharing(self):
        changed = (not hasattr(self, "attention_sharing")
                   or not hasattr(self.config, "sharing_lookup_path")
                   or self.config.sharing_lookup_path != config.sharing_lookup_path)
        if changed:
            self.attention_sharing = AttentionSharing(config.sharing_lookup_path)
        else:
            self.attention_sharing.reset_state()
        for knob in ("sharing_lookup_path", "pattern_threshold", "similarity_threshold",
                     "fallback_threshold", "block_size", "min_budget", "max_budget",
                     "queryaware_threshold"):
            setattr(self.config, knob, getattr(config, knob))
        sharing = self.attention_sharing

        def point_at_state(m):
            if isinstance(m, Attention):
                m.attention_sharing = sharing

        self.apply(point_at_state)
        return sharing

    model.__class__._init_attention_sharing = _init_attention_sharing
    model.__class__.reset_attention_sharing = reset_attention_sharing
    model.attention_sharing = model._init_attention_sharing()
    model.model._use_sdpa = False

    original = model.forward.__func__

    @functools.wraps(original)
    def forward_with_reset(self, *args, **kwargs):
        # a kernel of the previous forward that gave up on a bounded wait left rows unwritten: say so
        # here, where a synchronisation costs nothing (the previous forward's result has been used)
        native.raise_on_device_timeouts()
        self.reset_attention_sharing()
        return original(self, *args, **kwargs)

    model.forward = forward_with_reset.__get__(model, model.__class__)
    LOGGER.info("Patched model for shareprefill.")
    return model
