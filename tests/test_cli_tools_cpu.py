"""The model store (pull / list / rm / show / resolve) and the checkpoint sub-commands of the CLI, on CPU."""
import json
import os

import pytest

from fllm_b200 import hub
from fllm_b200.cli import main as cli


@pytest.fixture()
def store(tmp_path, monkeypatch):
    monkeypatch.setenv("FLLM_HOME", str(tmp_path / "home"))
    return tmp_path


def _tiny_gguf(path):
    from fllm_b200.cpu_engine import write_tiny_llama_gguf
    write_tiny_llama_gguf(str(path))
    return str(path)


def test_store_pull_list_show_resolve_rm(store, capsys):
    src = _tiny_gguf(store / "tiny.gguf")
    e = hub.pull(src, name="tiny")
    assert e["name"] == "tiny" and os.path.exists(e["path"]) and e["bytes"] > 0
    with pytest.raises(hub.HubError):
        hub.pull(src, name="tiny")                        # already there
    assert [m["name"] for m in hub.list_models()] == ["tiny"]
    assert hub.resolve("tiny") == e["path"] and hub.resolve(src) == src and hub.resolve("qwen3-8b") == "qwen3-8b"
    info = hub.show("tiny")
    assert info["format"] == "gguf" and info["architecture"] == "llama" and info["tensor_types"]["Q4_K"] > 0
    assert cli(["list"]) == 0 and "tiny" in capsys.readouterr().out
    assert cli(["show", "tiny"]) == 0 and json.loads(capsys.readouterr().out)["layers"] == 2
    assert cli(["rm", "tiny"]) == 0 and hub.list_models() == [] and not os.path.exists(e["path"])
    assert cli(["rm", "tiny"]) == 1


def test_references_and_offline_pull(store):
    assert hub.parse_ref("hf://Qwen/Qwen3-8B@main:model.gguf") == {"repo": "Qwen/Qwen3-8B", "revision": "main", "file": "model.gguf"}
    with pytest.raises(hub.HubError):
        hub.parse_ref("s3://bucket/x")
    with pytest.raises(hub.HubError) as ei:               # no network here: a clear error, not a hang or a traceback
        hub.pull("hf://fllm-b200-tests/does-not-exist")
    assert "cannot fetch" in str(ei.value)
    assert "qwen3-8b" in hub.catalog()
    json.dump({"mine": "hf://me/mine"}, open(os.path.join(hub.home(), "catalog.json"), "w"))
    assert hub.catalog()["mine"] == "hf://me/mine"


def test_cli_quantize_set_split_merge_and_ppl(store, capsys):
    src = _tiny_gguf(store / "tiny.gguf")
    q8 = str(store / "q8.gguf")
    assert cli(["quantize", src, q8, "Q8_0"]) == 0
    assert json.loads(capsys.readouterr().out)["tensors"]["Q8_0"] > 0
    named = str(store / "named.gguf")
    assert cli(["gguf-set", q8, named, "--set", 'general.name="renamed"', "--set", "fllm.x=3"]) == 0
    assert hub.show(named)["format"] == "gguf"
    capsys.readouterr()
    assert cli(["gguf-split", named, str(store / "sh"), "--max-tensors", "5"]) == 0
    shards = json.loads(capsys.readouterr().out)
    assert len(shards) > 1 and cli(["gguf-merge", shards[0], str(store / "merged.gguf")]) == 0
    text = store / "t.txt"
    text.write_text("hello world, hello again. " * 8)
    capsys.readouterr()
    assert cli(["ppl", "--model", src, "--device", "cpu", "--ctx", "128", "--kv-blocks", "32", "--file", str(text)]) == 0
    out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert out["tokens"] > 50 and out["perplexity"] > 1.0


def test_sanitizer_build_of_the_cpu_library_runs_clean():
    """AddressSanitizer + UBSan build of the native CPU engine / codecs: the CPU self-test in a child process."""
    from fllm_b200 import _build, selftest
    if not _build.sanitizer_runtime():
        import pytest
        pytest.skip("no AddressSanitizer runtime with this compiler")
    assert selftest.selftest_sanitize() == 0
    assert _build.LIB_CPU_SAN.exists()
