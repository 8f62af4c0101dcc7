"""WARC records, HTML extraction, and the hashed n-gram classifiers as refinery stages."""
import gzip

from openagents_b200.data.classifiers import HashedNgramClassifier, classifier_stage
from openagents_b200.data.extract import html_to_text, iter_warc_records, warc_to_documents

HTML = b"""<!doctype html><html><head><meta charset="utf-8"><title>Mill &amp; Bridge</title><style>p{color:red}</style>
<script>var x = "<p>not text</p>";</script></head><body><h1>The old mill</h1><p>Grain&nbsp;comes   by <b>boat</b>.<br>Twice a week.</p>
<ul><li>na&iuml;ve caf&eacute;</li><li>second</li></ul><noscript>enable js</noscript></body></html>"""


def _warc(records):
    out = b""
    for typ, uri, body in records:
        head = f"WARC/1.0\r\nWARC-Type: {typ}\r\nWARC-Target-URI: {uri}\r\nWARC-Date: 2026-01-01T00:00:00Z\r\nContent-Length: {len(body)}\r\n\r\n".encode()
        out += head + body + b"\r\n\r\n"
    return out


def test_html_extraction_keeps_text_and_structure():
    text = html_to_text(HTML)
    assert text.split("\n") == ["Mill & Bridge", "The old mill", "Grain comes by boat.", "Twice a week.", "naïve café", "second"]
    assert "not text" not in text and "color:red" not in text and "enable js" not in text
    assert html_to_text("<p>unclosed <b>tags <i>everywhere") == "unclosed tags everywhere"
    assert html_to_text(b"<p>caf\xe9</p>") == "café"                    # not UTF-8: falls back to Latin-1


def test_warc_records_plain_and_gzip_and_truncated():
    http = b"HTTP/1.1 200 OK\r\nContent-Type: text/html; charset=UTF-8\r\n\r\n" + HTML
    gone = b"HTTP/1.1 404 Not Found\r\nContent-Type: text/html\r\n\r\n<p>" + b"missing " * 20 + b"</p>"
    pdf = b"HTTP/1.1 200 OK\r\nContent-Type: application/pdf\r\n\r\n%PDF" + b"x" * 100
    blob = _warc([("warcinfo", "", b"software: test"), ("response", "http://a.example/mill", http), ("request", "http://a.example/mill", b"GET /"),
                  ("response", "http://a.example/gone", gone), ("response", "http://a.example/doc.pdf", pdf)])
    recs = list(iter_warc_records(blob))
    assert [r["uri"] for r in recs] == ["http://a.example/mill", "http://a.example/gone", "http://a.example/doc.pdf"]
    assert recs[0]["httpStatus"] == 200 and recs[0]["contentType"] == "text/html" and recs[0]["charset"] == "UTF-8" and recs[0]["payload"] == HTML
    assert len(list(iter_warc_records(blob, types=("response", "request", "warcinfo")))) == 5
    docs = warc_to_documents(gzip.compress(blob[:len(blob) // 2]) + gzip.compress(blob[len(blob) // 2:]))       # two gzip members
    assert len(docs) == 1 and docs[0]["uri"] == "http://a.example/mill" and docs[0]["lines"][1] == "The old mill"
    assert [r["uri"] for r in iter_warc_records(blob[:-150])] == ["http://a.example/mill", "http://a.example/gone"]     # a cut file ends quietly


def test_language_id_and_quality_classifier_as_refinery_stages(tmp_path):
    en = ["the river runs north past the old mill", "boats carry grain to the market every week", "she said that it was the best of times",
          "where is the nearest station and when does the train leave", "this is a short sentence about the weather today"]
    de = ["der fluss fliesst nach norden an der alten muehle vorbei", "boote bringen jede woche getreide zum markt", "sie sagte dass es die beste aller zeiten war",
          "wo ist der naechste bahnhof und wann faehrt der zug ab", "das ist ein kurzer satz ueber das wetter von heute"]
    fr = ["la riviere coule vers le nord pres du vieux moulin", "les bateaux apportent le grain au marche chaque semaine", "elle a dit que c'etait le meilleur des temps",
          "ou est la gare la plus proche et quand part le train", "ceci est une courte phrase sur le temps qu'il fait aujourd'hui"]
    lid = HashedNgramClassifier.fit(en + de + fr, ["en"] * 5 + ["de"] * 5 + ["fr"] * 5, epochs=40, buckets=1 << 13)
    assert lid.predict("the train to the market leaves when the weather is good")[0] == "en"
    assert lid.predict("der zug zum markt faehrt ab wenn das wetter gut ist")[0] == "de"
    assert lid.predict("le train pour le marche part quand il fait beau")[0] == "fr"
    lid.save(str(tmp_path / "lid.json"))
    again = HashedNgramClassifier.load(str(tmp_path / "lid.json"))
    assert again.predict("wo ist der markt")[0] == "de" and abs(again.predict("wo ist der markt")[1] - lid.predict("wo ist der markt")[1]) < 1e-5
    docs = [{"documentRef": "d.en", "lines": ["the boats leave the station every week"]}, {"documentRef": "d.de", "lines": ["die boote fahren jede woche vom bahnhof ab"]}]
    kept, rep = classifier_stage(docs, lid, "en", 0.4, stage="language_id")
    assert [d["documentRef"] for d in kept] == ["d.en"] and rep["rejected"] == {"de": 1} and rep["stage"] == "language_id"
    good = ["the committee reviewed the proposal and published a detailed report on the findings", "researchers measured the flow of the river over several seasons and compared the results",
            "the museum opened a new exhibition about the history of the grain trade in the region", "a careful reading of the text shows how the argument develops from its premises"]
    spam = ["buy now!!! click here $$$ free free free win big prizes now", "cheap pills best price click click click order now!!!", "win $$$ now!!! free bonus click here limited offer!!!",
            "hot deals!!! click now free free $$$ subscribe win win win"]
    q = HashedNgramClassifier.fit(good + spam, ["keep"] * 4 + ["drop"] * 4, epochs=60, buckets=1 << 13)
    kept, rep = classifier_stage([{"documentRef": "a", "lines": ["the report compared the results of several seasons of careful measurement"]},
                                  {"documentRef": "b", "lines": ["click here now!!! free $$$ prizes win win"]}], q, "keep", 0.5)
    assert [d["documentRef"] for d in kept] == ["a"] and rep["keptDocuments"] == 1 and rep["rejected"] == {"drop": 1}


def test_prepare_takes_crawl_files_and_a_language_filter(tmp_path, capsys):
    import json
    from openagents_b200.data.__main__ import main
    en = [f"the river number {i} runs north past the old mill and the boats carry grain to the market every week" for i in range(12)]
    de = [f"der fluss nummer {i} fliesst nach norden an der alten muehle vorbei und boote bringen getreide zum markt" for i in range(12)]
    lid = HashedNgramClassifier.fit(en[:6] + de[:6], ["en"] * 6 + ["de"] * 6, epochs=40, buckets=1 << 12)
    lid.save(str(tmp_path / "lid.json"))
    pages = [("response", f"http://x.example/{i}", b"HTTP/1.1 200 OK\r\nContent-Type: text/html\r\n\r\n<html><body><p>" + t.encode() + b"</p></body></html>")
             for i, t in enumerate(en[6:] + de[6:])]
    (tmp_path / "crawl.warc.gz").write_bytes(gzip.compress(_warc(pages)))
    assert main(["prepare", "--text", str(tmp_path / "crawl.warc.gz"), "--out", str(tmp_path / "o"), "--merges", "20", "--no-refine", "--val-fraction", "0",
                 "--language-id", f"{tmp_path / 'lid.json'}:en:0.5"]) == 0
    capsys.readouterr()
    man = json.loads((tmp_path / "o" / "manifest.json").read_text())
    assert man["refinery"]["inputDocuments"] == 12 and man["documents"] == 6
    assert man["refinery"]["stages"][-1]["stage"] == "language_id" and man["refinery"]["stages"][-1]["stats"]["rejected"] == {"de": 6}
