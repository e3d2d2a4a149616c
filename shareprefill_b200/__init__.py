"""B200-native sparse-prefill attention behind the ``SharePrefill(...)(model)`` patch API."""
from .patch import SharePrefill

__all__ = ["SharePrefill"]
