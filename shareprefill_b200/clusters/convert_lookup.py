"""Convert a head-cluster lookup in the reference's JSON layout
(``{"clusters": {id: [[layer, head], ...]}, "shared_clusters": [id, ...]}``,
attn/attention_sharing.py:368-378) into the compact table this package ships:

    {"format": "spf-cluster-table-v1", "num_layers": L, "num_heads": H,
     "cluster_of": [[cluster id per head] per layer], "shared_clusters": [ids]}

    python -m shareprefill_b200.clusters.convert_lookup IN.json OUT.json

Both layouts are accepted wherever a ``sharing_lookup_path`` is given.
"""
import json
import sys


def to_table(lookup: dict) -> dict:
    pairs = [(int(l), int(h), cid) for cid, lst in lookup["clusters"].items() for l, h in lst]
    n_layers = max(p[0] for p in pairs) + 1
    n_heads = max(p[1] for p in pairs) + 1
    table = [[None] * n_heads for _ in range(n_layers)]
    for l, h, cid in pairs:
        if table[l][h] is None:  # the reference returns the first cluster that lists the pair
            table[l][h] = cid
    return {"format": "spf-cluster-table-v1", "num_layers": n_layers, "num_heads": n_heads,
            "cluster_of": table, "shared_clusters": list(lookup["shared_clusters"])}


def from_table(table: dict) -> dict:
    clusters = {}
    for l, row in enumerate(table["cluster_of"]):
        for h, cid in enumerate(row):
            if cid is not None:
                clusters.setdefault(str(cid), []).append([l, h])
    return {"clusters": clusters, "shared_clusters": [str(c) for c in table["shared_clusters"]]}


if __name__ == "__main__":
    with open(sys.argv[1]) as f:
        src = json.load(f)
    with open(sys.argv[2], "w") as f:
        json.dump(to_table(src), f, separators=(",", ":"))
