"""Model basename -> shipped head-cluster table (relative to the package directory).

Mirrors SHARING_LOOKUP_REGISTRY (clusters/sharing_lookup_registry.py:15-19); the table is the
reference's Llama-3.1-8B-Instruct lookup converted by ``convert_lookup.py``.
"""
SHARING_LOOKUP_REGISTRY = {
    "Llama-3.1-8B-Instruct": "clusters/llama31_8b_instruct_table.json",
}
