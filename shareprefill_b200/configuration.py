"""Knobs of the sparse-prefill patch.

Mirrors ``SharePrefillConfig`` (shareprefill_configurations.py:28-72): same constructor
arguments, defaults and attributes.  One deliberate difference: the reference splits
``model_name`` before looking at ``sharing_lookup_path`` (:67-69) and so raises on
``model_name=None`` even when an explicit lookup path is given; here an explicit path
is enough.
"""
from __future__ import annotations

import os
from pathlib import Path
from typing import Optional

from .clusters.registry import SHARING_LOOKUP_REGISTRY

BASE_DIR = Path(__file__).resolve().parent


class SharePrefillConfig:
    SUPPORTED_ATTENTION_TYPES = ["shareprefill"]

    def __init__(
        self,
        attn_type: str = "shareprefill",
        model_name: Optional[str] = None,
        sharing_lookup_path: Optional[str] = None,
        pattern_threshold: float = 0.9,
        similarity_threshold: float = 0.5,
        fallback_threshold: float = 0.9,
        queryaware_threshold: float = 0.1,
        block_size: int = 128,
        min_budget: Optional[int] = 1024,
        max_budget: Optional[int] = None,
        **kwargs,
    ):
        assert attn_type in self.SUPPORTED_ATTENTION_TYPES, \
            f"The attention_type {attn_type} you specified is not supported."
        self.attn_type = attn_type
        self.sharing_lookup_path = self.update_sharing_lookup_path(sharing_lookup_path, model_name)
        self.model_name = model_name
        self.pattern_threshold = pattern_threshold
        self.similarity_threshold = similarity_threshold
        self.fallback_threshold = fallback_threshold
        self.block_size = block_size
        self.min_budget = min_budget
        self.max_budget = max_budget
        self.queryaware_threshold = queryaware_threshold

    @classmethod
    def _resolve_sharing_lookup_path(cls, model_key: str) -> str:
        if model_key not in SHARING_LOOKUP_REGISTRY:
            raise AssertionError(f"Unsupported model {model_key}. ")
        return os.path.join(BASE_DIR, SHARING_LOOKUP_REGISTRY[model_key])

    @classmethod
    def update_sharing_lookup_path(cls, sharing_lookup_path: Optional[str], model_name: Optional[str]):
        if sharing_lookup_path is not None:
            return sharing_lookup_path
        if model_name is None:
            raise AssertionError("Unsupported model None. ")
        return cls._resolve_sharing_lookup_path(model_name.split("/")[-1])

    @classmethod
    def get_available_attn_types(cls):
        return cls.SUPPORTED_ATTENTION_TYPES
