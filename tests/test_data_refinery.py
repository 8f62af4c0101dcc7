"""The refinery as a pipeline, trace conversion and the ``prepare`` command."""
import json

from openagents_b200.data import ByteBpe, TokenDataset
from openagents_b200.data.__main__ import main
from openagents_b200.data.refinery import documents_from_texts, refine
from openagents_b200.data.traces import traces_to_records
from openagents_b200.oracle import cs336_more as a4

GOOD = ["The river runs north past the old mill and the stone bridge.\nBoats carry grain to the market town every week.\nAll rights reserved by nobody.",
        "A kettle of soup needs onions, carrots, salt and a slow fire.\nWrite to cook@example.org or call 555-0123 for the recipe.\nAll rights reserved by nobody.",
        "### $$$ %% @@ ^^ && ** (( )) -- ++ == ~~ ## !!\n%% ^^ && ** (( ))",
        "The river runs north past the old mill and the stone bridge.\nBoats carry grain to the market town every week.\nAnd sometimes barley too."]


def test_pipeline_masks_dedups_filters_and_reports():
    docs, rep = refine(documents_from_texts(GOOD))
    stages = {s["stage"]: s for s in rep["stages"]}
    assert stages["pii_masking"]["stats"]["maskedEmails"] == 1 and stages["pii_masking"]["stats"]["maskedPhones"] == 1
    text = "\n".join("\n".join(d["lines"]) for d in docs)
    assert "[EMAIL]" in text and "example.org" not in text
    assert text.count("All rights reserved") == 1                       # boilerplate kept once
    assert stages["gopher_rules"]["stats"]["rejectedSymbolHeavy"] + stages["gopher_rules"]["stats"]["rejectedLowAlphaRatio"] >= 1
    assert all("$$$" not in ln for d in docs for ln in d["lines"])
    assert rep["outputDocuments"] == len(docs) < rep["inputDocuments"] and rep["outputDigest"].startswith("sha256:")
    again, rep2 = refine(documents_from_texts(GOOD))
    assert rep2["outputDigest"] == rep["outputDigest"]
    # the reference corpus through the same chain: near duplicates (every fourth document) go away
    synth = a4.build_synthetic_corpus("ab" * 32, 32, 6)
    kept, r = refine(synth, stages=("minhash_dedup",), seed="ab" * 32)
    want, _ = a4.minhash_dedup(synth, "ab" * 32)
    assert [d["documentRef"] for d in kept] == want and len(kept) < 32


def test_traces_become_masked_records_with_reasons():
    def tr(answer, finish="stop", outcome=None, msgs=None, **extra):
        t = {"messages": msgs or [{"role": "system", "content": "Be brief."}, {"role": "user", "content": "Mail me at a@b.io please"}],
             "response": {"choices": [{"message": {"role": "assistant", "content": answer, **extra}, "finish_reason": finish}]}}
        if outcome:
            t["outcome"] = outcome
        return t
    tool_msgs = [{"role": "user", "content": "Weather in Oslo?"},
                 {"role": "assistant", "content": None, "tool_calls": [{"id": "c1", "type": "function", "function": {"name": "weather", "arguments": "{\"city\": \"Oslo\"}"}}]},
                 {"role": "tool", "tool_call_id": "c1", "content": "4 C, rain"}]
    traces = [tr("Sure."), tr("Sure."), tr("cut off", finish="length"), tr("bad", outcome="rejected"), tr("   "), {"messages": []},
              tr("Cold and wet.", msgs=tool_msgs), tr("x" * 300)]
    recs, rep = traces_to_records(traces, max_chars=200)
    assert rep["records"] == 2 and rep["dropped"] == {"rejected_outcome": 1, "unfinished_answer": 1, "empty_answer": 1, "malformed": 1, "duplicate": 1, "too_long": 1}
    assert recs[0]["messages"][1]["content"] == "Mail me at [EMAIL] please" and rep["maskedSpans"] == 1
    roles = [m["role"] for m in recs[1]["messages"]]
    assert roles == ["user", "assistant", "user", "assistant"]
    assert '[tool call] {"arguments": {"city": "Oslo"}, "name": "weather"}' in recs[1]["messages"][1]["content"]
    assert recs[1]["messages"][2]["content"].startswith("[tool result c1]")
    # the records are what the instruction-tuning lane takes
    from openagents_b200.train import sft
    tok = ByteBpe.train(b"Cold and wet. Weather in Oslo? Sure.", 8, special=sft.SPECIAL_TOKENS)
    assert sft.build_corpus(recs, tok, "traces@v1").manifest["recordCount"] == 2


def test_prepare_writes_shards_tokenizer_and_manifest(tmp_path, capsys):
    src = tmp_path / "c.txt"
    src.write_text("\n\n".join(GOOD * 3 + [f"Document number {i} talks about rivers, boats and the grain market in town {i}." for i in range(40)]))
    jl = tmp_path / "d.jsonl"
    jl.write_text(json.dumps({"text": "A separate note about bridges and mills along the northern river."}) + "\n")
    assert main(["prepare", "--text", str(src), str(jl), "--out", str(tmp_path / "o"), "--merges", "50", "--val-fraction", "0.1", "--shard-tokens", "400"]) == 0
    out = json.loads(capsys.readouterr().out)
    man = json.loads((tmp_path / "o" / "manifest.json").read_text())
    assert man["trainTokens"] == out["trainTokens"] > 400 and man["valTokens"] > 0 and man["bytesPerToken"] > 1.5
    assert man["refinery"]["inputDocuments"] == 53 and man["documents"] < 53
    train = sorted(p for p in (tmp_path / "o").iterdir() if p.name.startswith("train-"))
    assert len(train) == -(-man["trainTokens"] // 400)
    ds = TokenDataset(train, seq_len=32)
    assert ds.tokens == man["trainTokens"]
    tok = ByteBpe.from_json((tmp_path / "o" / "tokenizer.json").read_text())
    assert tok.vocab_size == man["vocabSize"] == 256 + 50 + 1
    first = ds.window(0)[0].tolist()
    assert tok.decode(first).startswith(("The river", "A kettle", "Document", "A separate"))
    # traces sub-command
    tj = tmp_path / "t.jsonl"
    tj.write_text(json.dumps({"messages": [{"role": "user", "content": "hi"}], "response": {"choices": [{"message": {"role": "assistant", "content": "hello"}, "finish_reason": "stop"}]}}) + "\n")
    assert main(["traces", "--in", str(tj), "--out", str(tmp_path / "r.jsonl")]) == 0
    assert json.loads((tmp_path / "r.jsonl").read_text())["messages"][-1] == {"role": "assistant", "content": "hello"}
