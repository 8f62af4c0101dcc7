"""Raw crawl bytes -> text: WARC response records and HTML extraction.

The reference's continuation audit lists the stages of the course's data assignment that its upstream refinery had not
landed yet: HTML extraction from WARC bytes, language identification and model-backed quality classifiers
(docs/2026-06-10-cs336-distributed-homework-continuation-audit.md:280-295).  This module is the first of them, on the
standard library only: ``iter_warc_records`` walks an (optionally gzip-compressed, possibly multi-member) WARC file and yields
the HTTP response records; ``html_to_text`` drops scripts, styles and markup, keeps block structure as line breaks, decodes
entities and normalises white space.
"""
from __future__ import annotations

import gzip
import io
import re
from html.parser import HTMLParser

_BLOCK = {"p", "div", "br", "li", "ul", "ol", "tr", "table", "h1", "h2", "h3", "h4", "h5", "h6", "section", "article", "header", "footer",
          "blockquote", "pre", "hr", "title", "dd", "dt", "figcaption", "option"}
_SKIP = {"script", "style", "noscript", "template", "svg", "head", "iframe", "object", "canvas"}


class _Text(HTMLParser):
    def __init__(self):
        super().__init__(convert_charrefs=True)
        self.out: list[str] = []
        self.skip = 0
        self.title: str | None = None
        self._in_title = False

    def handle_starttag(self, tag, attrs):
        if tag == "title":                      # the title sits inside <head>, which is otherwise skipped
            self._in_title = True
            return
        if tag in _SKIP:
            self.skip += 1
        elif tag in _BLOCK:
            self.out.append("\n")

    def handle_endtag(self, tag):
        if tag == "title":
            self._in_title = False
            return
        if tag in _SKIP:
            self.skip = max(0, self.skip - 1)
        elif tag in _BLOCK:
            self.out.append("\n")

    def handle_data(self, data):
        if self._in_title:
            self.title = (self.title or "") + data
        elif not self.skip:
            self.out.append(data)


def decode_bytes(raw: bytes, declared: str | None = None) -> str:
    """Bytes -> str by the declared charset, a ``<meta charset>`` in the first kilobytes, UTF-8, then Latin-1."""
    cands = []
    if declared:
        cands.append(declared)
    m = re.search(rb"charset=[\"']?([A-Za-z0-9_.:-]+)", raw[:4096], re.I)
    if m:
        cands.append(m.group(1).decode("ascii", "replace"))
    for enc in cands + ["utf-8"]:
        try:
            return raw.decode(enc)
        except (UnicodeDecodeError, LookupError):
            continue
    return raw.decode("latin-1")


def html_to_text(html: str | bytes, keep_title: bool = True) -> str:
    if isinstance(html, (bytes, bytearray)):
        html = decode_bytes(bytes(html))
    p = _Text()
    try:
        p.feed(html)
        p.close()
    except Exception:      # noqa: BLE001 - malformed markup: keep what was extracted so far
        pass
    text = "".join(p.out)
    lines = [re.sub(r"[ \t\r\f\v ]+", " ", ln).strip() for ln in text.split("\n")]
    lines = [ln for ln in lines if ln]
    if keep_title and p.title and p.title.strip():
        lines.insert(0, re.sub(r"\s+", " ", p.title).strip())
    return "\n".join(lines)


def _open_maybe_gzip(path_or_bytes) -> io.BufferedIOBase:
    raw = open(path_or_bytes, "rb") if isinstance(path_or_bytes, (str, bytes.__class__)) and not isinstance(path_or_bytes, (bytes, bytearray)) else io.BytesIO(path_or_bytes)
    head = raw.read(2)
    raw.seek(0)
    return gzip.GzipFile(fileobj=raw) if head == b"\x1f\x8b" else raw          # GzipFile reads concatenated members as one stream


def iter_warc_records(path_or_bytes, types=("response",)):
    """Yields ``{"type", "uri", "date", "httpStatus", "contentType", "charset", "payload"}`` for each record of the wanted types.  A record
    that cannot be parsed ends the iteration quietly at that point (truncated crawl files are common)."""
    f = _open_maybe_gzip(path_or_bytes)
    while True:
        line = f.readline()
        if not line:
            return
        if not line.startswith(b"WARC/"):
            continue
        headers = {}
        while True:
            h = f.readline()
            if not h or h in (b"\r\n", b"\n"):
                break
            k, _, v = h.partition(b":")
            headers[k.strip().lower().decode("latin-1")] = v.strip().decode("utf-8", "replace")
        try:
            n = int(headers.get("content-length", ""))
        except ValueError:
            return
        body = f.read(n)
        if len(body) < n:
            return
        if headers.get("warc-type") not in types:
            continue
        rec = {"type": headers.get("warc-type"), "uri": headers.get("warc-target-uri"), "date": headers.get("warc-date"), "httpStatus": None,
               "contentType": None, "charset": None, "payload": body}
        if headers.get("warc-type") == "response" and body.startswith(b"HTTP/"):
            head, sep, payload = body.partition(b"\r\n\r\n")
            if not sep:
                head, sep, payload = body.partition(b"\n\n")
            lines = head.split(b"\n")
            parts = lines[0].split()
            rec["httpStatus"] = int(parts[1]) if len(parts) > 1 and parts[1].isdigit() else None
            for ln in lines[1:]:
                k, _, v = ln.partition(b":")
                if k.strip().lower() == b"content-type":
                    ct = v.strip().decode("latin-1")
                    rec["contentType"] = ct.split(";")[0].strip().lower()
                    m = re.search(r"charset=([A-Za-z0-9_.:-]+)", ct, re.I)
                    rec["charset"] = m.group(1) if m else None
            rec["payload"] = payload
        yield rec


def warc_to_documents(path_or_bytes, min_chars: int = 50) -> list[dict]:
    """HTML responses with status 200 -> ``{"documentRef", "uri", "lines"}`` for the refinery."""
    docs = []
    for i, r in enumerate(iter_warc_records(path_or_bytes)):
        if r["httpStatus"] != 200 or (r["contentType"] or "text/html") not in ("text/html", "application/xhtml+xml"):
            continue
        text = html_to_text(decode_bytes(r["payload"], r["charset"]))
        if len(text) >= min_chars:
            docs.append({"documentRef": f"warc.{i}", "uri": r["uri"], "lines": text.split("\n")})
    return docs
