"""BERT-family encoder: hidden states and classification logits against Hugging Face `transformers` on a random
tiny checkpoint (packed batch of ragged sequences), pooling, and the HTTP surface of the encoder server."""
import pytest
import torch

transformers = pytest.importorskip("transformers")


def _tiny_bert(tmp_path, roberta=False, labels=1):
    torch.manual_seed(0)
    if roberta:
        from transformers import RobertaConfig, RobertaForSequenceClassification
        hc = RobertaConfig(vocab_size=300, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, intermediate_size=128,
                           max_position_embeddings=66, pad_token_id=1, num_labels=labels, type_vocab_size=1)
        m = RobertaForSequenceClassification(hc).eval()
    else:
        from transformers import BertConfig, BertForSequenceClassification
        hc = BertConfig(vocab_size=300, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, intermediate_size=128,
                        max_position_embeddings=64, num_labels=labels)
        m = BertForSequenceClassification(hc).eval()
    d = str(tmp_path / ("roberta" if roberta else "bert"))
    m.save_pretrained(d, safe_serialization=True)
    return m, d


@pytest.mark.parametrize("roberta", [False, True])
def test_encoder_matches_transformers(tmp_path, roberta):
    from fllm_b200.models.encoder import Encoder, load_hf_encoder
    from fllm_b200.ops.reference import RefOps
    m, d = _tiny_bert(tmp_path, roberta, labels=3)
    cfg, w = load_hf_encoder(d, "cpu", torch.float32)
    assert cfg.num_labels == 3 and cfg.arch == ("roberta" if roberta else "bert")
    enc = Encoder(cfg, w, RefOps(), "cpu")
    seqs = [[101, 5, 6, 7, 102], [101, 9, 10, 11, 12, 13, 14, 102, 20, 21, 22, 102], [7] * 33]
    types = [[0] * 5, [0] * 8 + ([0] * 4 if roberta else [1] * 4), [0] * 33]
    x = enc.forward(seqs, types)
    base = m.roberta if roberta else m.bert
    at = 0
    with torch.no_grad():
        for s, ty in zip(seqs, types):
            ref = base(torch.tensor([s]), token_type_ids=torch.tensor([ty])).last_hidden_state[0]
            assert (x[at:at + len(s)] - ref).abs().max().item() < 1e-4
            at += len(s)
        want = torch.stack([m(torch.tensor([s]), token_type_ids=torch.tensor([ty])).logits[0] for s, ty in zip(seqs, types)])
    assert (enc.classify(seqs, types) - want).abs().max().item() < 1e-4
    e_cls = enc.embed(seqs, types)
    e_mean = enc.embed(seqs, types, pooling="mean", normalize=False)
    assert e_cls.shape == (3, 64) and torch.allclose(e_cls.norm(dim=-1), torch.ones(3), atol=1e-5)
    assert torch.allclose(e_mean[0], x[:5].float().mean(0), atol=1e-5)
    with pytest.raises(ValueError):
        enc.forward([[1] * 100])


def test_encoder_server_routes(tmp_path):
    from fastapi.testclient import TestClient
    from fllm_b200.models.encoder import Encoder, load_hf_encoder
    from fllm_b200.ops.reference import RefOps
    from fllm_b200.server.encoder_app import EncoderService, create_encoder_app
    from fllm_b200.tokenizer import ByteTokenizer
    m, d = _tiny_bert(tmp_path, labels=1)
    cfg, w = load_hf_encoder(d, "cpu", torch.float32)
    svc = EncoderService(Encoder(cfg, w, RefOps(), "cpu"), ByteTokenizer(cfg.vocab_size), max_batch_tokens=24)
    c = TestClient(create_encoder_app(svc, "tiny-bert"))
    assert c.get("/health").json()["status"] == "ok"
    assert c.get("/v1/models").json()["data"][0]["task"] == "classify"
    r = c.post("/v1/embeddings", json={"input": ["hello world", "a", "third text here"]}).json()
    assert len(r["data"]) == 3 and len(r["data"][0]["embedding"]) == 64 and r["usage"]["prompt_tokens"] > 0
    one = c.post("/v1/embeddings", json={"input": "hello world"}).json()["data"][0]["embedding"]
    assert max(abs(a - b) for a, b in zip(one, r["data"][0]["embedding"])) < 1e-5      # batching does not change a vector
    assert len(c.post("/embed", json={"inputs": ["x", "y"]}).json()) == 2
    assert len(c.post("/pooling", json={"input": "abc", "pooling": "mean"}).json()["data"][0]["data"]) == 64
    cl = c.post("/classify", json={"input": ["abc", "defg"]}).json()
    assert len(cl["data"]) == 2 and 0.0 <= cl["data"][0]["probs"][0] <= 1.0
    sc = c.post("/v1/score", json={"text_1": "query", "text_2": ["doc one", "doc two"]}).json()
    assert len(sc["data"]) == 2
    rr = c.post("/v1/rerank", json={"query": "query", "documents": ["doc one", "doc two", "doc three"], "top_n": 2,
                                    "return_documents": True}).json()
    assert len(rr["results"]) == 2 and rr["results"][0]["relevance_score"] >= rr["results"][1]["relevance_score"]
    assert rr["results"][0]["document"]["text"].startswith("doc")
    want = {d["index"]: d["score"] for d in sc["data"]}
    for res in rr["results"]:
        if res["index"] in want:
            assert abs(res["relevance_score"] - want[res["index"]]) < 1e-5
    assert c.post("/v1/embeddings", json={"input": []}).status_code == 400
    assert c.post("/v1/rerank", json={"query": "q"}).status_code == 400
    assert c.post("/v1/embeddings", json={"input": "x" * 200}).status_code == 200        # truncated to the model's positions
