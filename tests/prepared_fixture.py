"""Writes a prepared-weights directory (manifest.json + data.bin) in the reference's format 1 (src/prepared.rs:15-50,
docs/ARTIFACTS.md "Prepared target"), for the loader tests.  Tensors are numpy arrays placed in a nested python structure
of dicts (objects), lists (sequences) and ("dict", [(key, value), ...]) nodes."""
import hashlib
import json
import os

import numpy as np

DTYPES = {np.dtype(np.int32): "int32", np.dtype(np.uint32): "int32", np.dtype(np.float16): "float16", np.dtype(np.float32): "float32",
          np.dtype(np.uint8): "uint8", np.dtype(np.int64): "int64"}


def write_prepared(directory, tree, key, chunk=1 << 16, object_tag="tensorfold.families.glm5_next.cuda.weights:Weights", align=256,
                   cpu_paths=()):
    """tree: the python structure; returns the manifest path.  Every tensor gets its own storage (aligned to `align`)."""
    os.makedirs(directory, exist_ok=True)
    payload = bytearray()
    storages = []

    def node(v, path):
        if isinstance(v, np.ndarray):
            a = np.ascontiguousarray(v)
            while len(payload) % align:
                payload.append(0)
            dev = "cpu" if path in cpu_paths else "cuda"
            storages.append({"offset": len(payload), "nbytes": a.nbytes, "dev": dev})
            payload.extend(a.tobytes())
            stride, s = [], 1
            for n in reversed(a.shape):
                stride.insert(0, s)
                s *= n
            return {"T": len(storages) - 1, "dtype": DTYPES[a.dtype], "shape": list(a.shape), "stride": stride, "off": 0, "dev": dev}
        if isinstance(v, dict):
            return {"O": object_tag if path == "weights" else "object", "f": {k: node(x, f"{path}.{k}") for k, x in v.items()}}
        if isinstance(v, list):
            return {"L": [node(x, f"{path}[{i}]") for i, x in enumerate(v)]}
        if isinstance(v, tuple) and v[0] == "dict":
            return {"D": [[k, node(x, f"{path}[{json.dumps(k)}]")] for k, x in v[1]]}
        return {"P": v}
    tree_json = node(tree, "weights")
    data = bytes(payload)
    hashes = [hashlib.sha256(data[o:o + chunk]).hexdigest() for o in range(0, len(data), chunk)]
    manifest = {"format": 1, "file_size": len(data), "chunk": chunk, "chunk_sha256": hashes, "storages": storages, "tree": tree_json, "key": key}
    open(os.path.join(directory, "data.bin"), "wb").write(data)
    mp = os.path.join(directory, "manifest.json")
    json.dump(manifest, open(mp, "w"))
    return mp


def tp_shards(bank, world, experts):
    """Slices a bank of `experts` routed experts (the shared entry is dropped) the way the reference's tensor-parallel ranks
    hold it (src/experts.rs:146-156): gate/up columns, down rows and the intermediate-sized scale vectors cut `world` ways."""
    out = []
    I = bank["svh_g"].shape[1]
    Ir = I // world
    for r in range(world):
        sl = slice(r * Ir, (r + 1) * Ir)
        tl = slice(r * Ir // 16, (r + 1) * Ir // 16)
        out.append({"gt": bank["gt"][:experts, :, tl], "ut": bank["ut"][:experts, :, tl], "dt": bank["dt"][:experts, tl],
                    "suh_g": bank["suh_g"][:experts], "suh_u": bank["suh_u"][:experts], "suh_d": bank["suh_d"][:experts, sl],
                    "svh_g": bank["svh_g"][:experts, sl], "svh_u": bank["svh_u"][:experts, sl], "svh_d": bank["svh_d"][:experts]})
    return out
