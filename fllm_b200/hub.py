"""Local model store, references and aliases: what ``pull`` / ``list`` / ``rm`` / ``show`` and
``--model NAME`` resolve through.

The reference keeps an immutable snapshot cache for ``hf://`` references, a convert-once cache and a
catalog of aliases (rust/engine/src/hub.rs, import.rs:1-8, catalog.rs). Here:

* the store is a directory (``$FLLM_HOME/models``, default ``~/.cache/fllm_b200/models``) with one entry
  per model - a GGUF file or a checkpoint directory - and an ``index.json`` that records where each
  entry came from;
* ``pull`` takes a local path (copied or linked in), or ``hf://org/name[@revision][:file]``, which is
  fetched with ``huggingface_hub`` when the machine has network access and fails with a clear message
  when it has not;
* ``resolve`` turns what the user typed - a path, a store entry, an alias from the catalog - into a
  path or a preset name that the loader understands.
"""
from __future__ import annotations

import json
import os
import re
import shutil
import time
from typing import Dict, List, Optional

_CATALOG = {          # short names -> references (extend with $FLLM_HOME/catalog.json)
    "qwen3-8b": "hf://Qwen/Qwen3-8B", "qwen3-0.6b": "hf://Qwen/Qwen3-0.6B", "llama3.1-8b": "hf://meta-llama/Llama-3.1-8B-Instruct",
    "llama3.2-1b": "hf://meta-llama/Llama-3.2-1B-Instruct", "gpt-oss-20b": "hf://openai/gpt-oss-20b",
    "gpt-oss-120b": "hf://openai/gpt-oss-120b", "mistral-7b": "hf://mistralai/Mistral-7B-Instruct-v0.3",
}


class HubError(RuntimeError):
    pass


def home() -> str:
    return os.environ.get("FLLM_HOME") or os.path.join(os.path.expanduser("~"), ".cache", "fllm_b200")


def store_dir() -> str:
    d = os.path.join(home(), "models")
    os.makedirs(d, exist_ok=True)
    return d


def _index_path() -> str:
    return os.path.join(store_dir(), "index.json")


def _load_index() -> Dict[str, dict]:
    try:
        return json.load(open(_index_path()))
    except (OSError, json.JSONDecodeError):
        return {}


def _save_index(idx: Dict[str, dict]) -> None:
    tmp = _index_path() + ".tmp"
    json.dump(idx, open(tmp, "w"), indent=1)
    os.replace(tmp, _index_path())


def catalog() -> Dict[str, str]:
    out = dict(_CATALOG)
    try:
        out.update(json.load(open(os.path.join(home(), "catalog.json"))))
    except (OSError, json.JSONDecodeError):
        pass
    return out


def parse_ref(ref: str) -> dict:
    """``hf://org/name[@revision][:file]`` -> parts."""
    m = re.match(r"hf://([\w.\-]+/[\w.\-]+)(?:@([\w.\-]+))?(?::(.+))?$", ref)
    if not m:
        raise HubError(f"not a model reference: {ref!r} (expected hf://org/name[@revision][:file])")
    return {"repo": m.group(1), "revision": m.group(2), "file": m.group(3)}


def _safe_name(s: str) -> str:
    return re.sub(r"[^\w.\-]+", "--", s.strip("/")).strip("-") or "model"


def _size(path: str) -> int:
    if os.path.isfile(path):
        return os.path.getsize(path)
    return sum(os.path.getsize(os.path.join(r, f)) for r, _, fs in os.walk(path) for f in fs)


def pull(ref: str, name: Optional[str] = None, link: bool = False) -> dict:
    """Add a model to the store. Returns its index entry."""
    idx = _load_index()
    ref = catalog().get(ref, ref)
    if os.path.exists(ref):                                  # local file or directory
        src = os.path.abspath(ref)
        name = name or _safe_name(os.path.splitext(os.path.basename(src))[0] if os.path.isfile(src) else os.path.basename(src))
        dst = os.path.join(store_dir(), name + (".gguf" if os.path.isfile(src) and src.endswith(".gguf") else ""))
        if os.path.lexists(dst):
            raise HubError(f"{name!r} is already in the store (rm it first)")
        if link:
            os.symlink(src, dst)
        elif os.path.isfile(src):
            shutil.copy2(src, dst)
        else:
            shutil.copytree(src, dst)
        entry = {"name": name, "path": dst, "source": src, "added": int(time.time()), "bytes": _size(dst)}
    else:
        parts = parse_ref(ref)
        name = name or _safe_name(parts["repo"] + ("-" + parts["file"] if parts["file"] else ""))
        if name in idx:
            return idx[name]                                 # snapshots are immutable: a second pull is a no-op
        try:
            from huggingface_hub import hf_hub_download, snapshot_download
            target = os.path.join(store_dir(), name)
            if parts["file"]:
                got = hf_hub_download(parts["repo"], parts["file"], revision=parts["revision"], local_dir=target)
            else:
                got = snapshot_download(parts["repo"], revision=parts["revision"], local_dir=target,
                                        allow_patterns=["*.json", "*.safetensors", "*.gguf", "tokenizer.model", "*.txt"])
        except ImportError as e:
            raise HubError("downloading needs the huggingface_hub package") from e
        except Exception as e:                               # no network, no such repository, no permission
            raise HubError(f"cannot fetch {ref}: {type(e).__name__}: {e}") from e
        entry = {"name": name, "path": got, "source": ref, "added": int(time.time()), "bytes": _size(got)}
    idx[name] = entry
    _save_index(idx)
    return entry


def list_models() -> List[dict]:
    idx = _load_index()
    return [e for e in idx.values() if os.path.lexists(e["path"])]


def remove(name: str) -> bool:
    idx = _load_index()
    e = idx.pop(name, None)
    if e is None:
        return False
    p = e["path"]
    if os.path.islink(p) or os.path.isfile(p):
        os.remove(p)
    elif os.path.isdir(p):
        shutil.rmtree(p)
    _save_index(idx)
    return True


def resolve(name: str) -> str:
    """What to hand to the loader for `name`: an existing path stays; a store entry or alias that is in the store
    becomes its path; anything else (a preset name such as ``qwen3-8b`` with random weights) is returned as it is."""
    if os.path.exists(name):
        return name
    idx = _load_index()
    if name in idx and os.path.lexists(idx[name]["path"]):
        return idx[name]["path"]
    ref = catalog().get(name)
    if ref:
        for e in idx.values():
            if e.get("source") == ref and os.path.lexists(e["path"]):
                return e["path"]
    if name.startswith("hf://"):
        return pull(name)["path"]
    return name


def show(name: str) -> dict:
    """Facts about a stored model or a path: format, architecture, size, tensor types."""
    path = resolve(name)
    if not os.path.exists(path):
        raise HubError(f"no model {name!r} in the store and no such path")
    out = {"name": name, "path": path, "bytes": _size(path)}
    if path.endswith(".gguf"):
        from .formats.gguf import GgufReader
        r = GgufReader(path)
        arch = r.metadata.get("general.architecture", "?")
        types: Dict[str, int] = {}
        for t in r.tensors.values():
            types[t.type_name] = types.get(t.type_name, 0) + 1
        out.update(format="gguf", architecture=arch, tensors=len(r.tensors), tensor_types=types,
                   layers=r.metadata.get(f"{arch}.block_count"), context=r.metadata.get(f"{arch}.context_length"),
                   tokenizer="tokenizer.ggml.tokens" in r.metadata, chat_template="tokenizer.chat_template" in r.metadata)
        r.close()
    elif os.path.isdir(path) and os.path.exists(os.path.join(path, "config.json")):
        hf = json.load(open(os.path.join(path, "config.json")))
        out.update(format="safetensors", architecture=hf.get("model_type"), layers=hf.get("num_hidden_layers"),
                   hidden=hf.get("hidden_size"), vocab=hf.get("vocab_size"), quantization=(hf.get("quantization_config") or {}).get("quant_method"),
                   files=sorted(f for f in os.listdir(path) if f.endswith((".safetensors", ".json", ".model"))))
    else:
        out["format"] = "unknown"
    return out
