"""Event identity and signatures for the coordination records: Nostr event ids and BIP-340 Schnorr signatures over secp256k1.

The coordination protocol carries records and SIGNED pointers (docs/nips/TRN.md:25-31: receipts, verdicts and artifact locators
are events signed by the node that made them).  An event's id is the SHA-256 of the canonical serialisation
``[0, pubkey, created_at, kind, tags, content]`` (compact JSON, UTF-8), its signature a BIP-340 signature of that id under the
author's x-only public key.  Pure Python: the curve arithmetic is small, used a few times per training window, and has no
dependency; the implementation is checked against the standard's published test vectors (``tests/test_nostr.py``).
"""
from __future__ import annotations

import hashlib
import json

P = 0xFFFFFFFFFFFFFFFFFFFFFFFFFFFFFFFFFFFFFFFFFFFFFFFFFFFFFFFEFFFFFC2F
N = 0xFFFFFFFFFFFFFFFFFFFFFFFFFFFFFFFEBAAEDCE6AF48A03BBFD25E8CD0364141
G = (0x79BE667EF9DCBBAC55A06295CE870B07029BFCDB2DCE28D959F2815B16F81798, 0x483ADA7726A3C4655DA4FBFC0E1108A8FD17B448A68554199C47D08FFB10D4B8)


def _add(a, b):
    if a is None:
        return b
    if b is None:
        return a
    if a[0] == b[0] and (a[1] + b[1]) % P == 0:
        return None
    if a == b:
        lam = 3 * a[0] * a[0] * pow(2 * a[1], P - 2, P) % P
    else:
        lam = (b[1] - a[1]) * pow(b[0] - a[0], P - 2, P) % P
    x = (lam * lam - a[0] - b[0]) % P
    return (x, (lam * (a[0] - x) - a[1]) % P)


def _mul(pt, k: int):
    out = None
    while k:
        if k & 1:
            out = _add(out, pt)
        pt = _add(pt, pt)
        k >>= 1
    return out


def _tagged(tag: str, data: bytes) -> bytes:
    t = hashlib.sha256(tag.encode()).digest()
    return hashlib.sha256(t + t + data).digest()


def _lift_x(x: int):
    if x >= P:
        return None
    y2 = (pow(x, 3, P) + 7) % P
    y = pow(y2, (P + 1) // 4, P)
    if y * y % P != y2:
        return None
    return (x, y if y % 2 == 0 else P - y)


def public_key(seckey: bytes) -> bytes:
    """x-only public key (32 bytes) of a 32-byte secret key."""
    d = int.from_bytes(seckey, "big")
    if not 1 <= d < N:
        raise ValueError("secret key out of range")
    return _mul(G, d)[0].to_bytes(32, "big")


def schnorr_sign(msg: bytes, seckey: bytes, aux: bytes = b"\x00" * 32) -> bytes:
    d0 = int.from_bytes(seckey, "big")
    if not 1 <= d0 < N:
        raise ValueError("secret key out of range")
    if len(aux) != 32:
        raise ValueError("auxiliary randomness must be 32 bytes")
    Pt = _mul(G, d0)
    d = d0 if Pt[1] % 2 == 0 else N - d0
    t = (d ^ int.from_bytes(_tagged("BIP0340/aux", aux), "big")).to_bytes(32, "big")
    px = Pt[0].to_bytes(32, "big")
    k0 = int.from_bytes(_tagged("BIP0340/nonce", t + px + msg), "big") % N
    if k0 == 0:
        raise ValueError("nonce is zero")
    R = _mul(G, k0)
    k = k0 if R[1] % 2 == 0 else N - k0
    rx = R[0].to_bytes(32, "big")
    e = int.from_bytes(_tagged("BIP0340/challenge", rx + px + msg), "big") % N
    sig = rx + ((k + e * d) % N).to_bytes(32, "big")
    if not schnorr_verify(msg, px, sig):
        raise RuntimeError("the signature just made does not verify")
    return sig


def schnorr_verify(msg: bytes, pubkey: bytes, sig: bytes) -> bool:
    if len(pubkey) != 32 or len(sig) != 64:
        return False
    Pt = _lift_x(int.from_bytes(pubkey, "big"))
    r, s = int.from_bytes(sig[:32], "big"), int.from_bytes(sig[32:], "big")
    if Pt is None or r >= P or s >= N:
        return False
    e = int.from_bytes(_tagged("BIP0340/challenge", sig[:32] + pubkey + msg), "big") % N
    R = _add(_mul(G, s), _mul(Pt, N - e))
    return R is not None and R[1] % 2 == 0 and R[0] == r


def event_id(pubkey_hex: str, created_at: int, kind: int, tags: list, content: str) -> str:
    body = json.dumps([0, pubkey_hex, created_at, kind, tags, content], separators=(",", ":"), ensure_ascii=False)
    return hashlib.sha256(body.encode("utf-8")).hexdigest()


def finalize_event(event: dict, seckey: bytes, created_at: int, aux: bytes = b"\x00" * 32) -> dict:
    """An unsigned record (``kind``, ``tags``, ``content``) -> a signed event with ``pubkey``, ``created_at``, ``id`` and ``sig``."""
    pub = public_key(seckey).hex()
    eid = event_id(pub, created_at, event["kind"], event["tags"], event["content"])
    return {**event, "pubkey": pub, "created_at": created_at, "id": eid, "sig": schnorr_sign(bytes.fromhex(eid), seckey, aux).hex()}


def verify_event(event: dict) -> list[str]:
    """Problems of a signed event (empty = the id is the hash of the fields and the signature verifies under ``pubkey``)."""
    errs = []
    try:
        want = event_id(event["pubkey"], event["created_at"], event["kind"], event["tags"], event["content"])
        if want != event.get("id"):
            errs.append("id_mismatch")
        if not schnorr_verify(bytes.fromhex(want), bytes.fromhex(event["pubkey"]), bytes.fromhex(event.get("sig", ""))):
            errs.append("bad_signature")
    except (KeyError, ValueError, TypeError):
        errs.append("malformed_event")
    return errs
