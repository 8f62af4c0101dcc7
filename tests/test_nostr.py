"""BIP-340 signatures against the standard's test vectors, event ids, and signed coordination records."""
from openagents_b200.control import coordination as co
from openagents_b200.control import nostr

H = bytes.fromhex


def test_bip340_vectors():
    # index 0 of the standard's vector file
    sk = H("0000000000000000000000000000000000000000000000000000000000000003")
    pk = H("F9308A019258C31049344F85F89D5229B531C845836F99B08601F113BCE036F9")
    msg = H("00" * 32)
    sig = H("E907831F80848D1069A5371B402410364BDF1C5F8307B0084C55F1CE2DCA821525F66A4A85EA8B71E482A74F382D2CE5EBEEE8FDB2172F477DF4900D310536C0")
    assert nostr.public_key(sk) == pk
    assert nostr.schnorr_sign(msg, sk, H("00" * 32)) == sig
    assert nostr.schnorr_verify(msg, pk, sig)
    # index 1
    sk1 = H("B7E151628AED2A6ABF7158809CF4F3C762E7160F38B4DA56A784D9045190CFEF")
    pk1 = H("DFF1D77F2A671C5F36183726DB2341BE58FEAE1DA2DECED843240F7B502BA659")
    msg1 = H("243F6A8885A308D313198A2E03707344A4093822299F31D0082EFA98EC4E6C89")
    sig1 = H("6896BD60EEAE296DB48A229FF71DFE071BDE413E6D43F917DC8DCF8C78DE33418906D11AC976ABCCB20B091292BFF4EA897EFCB639EA871CFA95F6DE339E4B0A")
    assert nostr.public_key(sk1) == pk1
    assert nostr.schnorr_sign(msg1, sk1, H("0000000000000000000000000000000000000000000000000000000000000001")) == sig1
    assert nostr.schnorr_verify(msg1, pk1, sig1)
    # tampering: another message, a flipped signature bit, a key that is not on the curve
    assert not nostr.schnorr_verify(H("01" + "00" * 31), pk, sig)
    assert not nostr.schnorr_verify(msg, pk, sig[:-1] + bytes([sig[-1] ^ 1]))
    assert not nostr.schnorr_verify(msg, H("EEFDEA4CDB677750A420FEE807EACF21EB9898AE79B9768766E4FAA04A2D4A34"), sig)
    assert not nostr.schnorr_verify(msg, pk, sig[:32]) and not nostr.schnorr_verify(msg, pk[:31], sig)


def test_signed_coordination_records():
    sk = H("B7E151628AED2A6ABF7158809CF4F3C762E7160F38B4DA56A784D9045190CFEF")
    window = co.training_window("net.1", "window.7", 7, "checkpoint.round.7", 16, "policy.default")
    receipt = co.training_receipt(window, nostr.public_key(sk).hex(), 16, 16 * 512 * 1024, "artifact.delta.7", "sha256:" + "ab" * 32)
    assert co.check_event(receipt) == []
    ev = nostr.finalize_event(receipt, sk, created_at=1_780_000_000)
    assert nostr.verify_event(ev) == [] and len(ev["id"]) == 64 and len(ev["sig"]) == 128 and ev["pubkey"] == nostr.public_key(sk).hex()
    assert ev["id"] == nostr.event_id(ev["pubkey"], ev["created_at"], ev["kind"], ev["tags"], ev["content"])
    forged = {**ev, "content": ev["content"].replace("16", "17", 1)}
    assert forged["content"] != ev["content"] and nostr.verify_event(forged) == ["id_mismatch", "bad_signature"]
    # a verdict that points at the receipt by its id
    verdict = nostr.finalize_event(co.validator_verdict(window, ev["id"], ev["pubkey"], "accepted"), H("00" * 31 + "03"), created_at=1_780_000_100)
    assert nostr.verify_event(verdict) == [] and co.first_tag(verdict, "e") == ev["id"]
    moved = {**ev, "created_at": ev["created_at"] + 1}
    assert "id_mismatch" in nostr.verify_event(moved)
    resigned_by_other = {**ev, "pubkey": nostr.public_key(H("00" * 31 + "03")).hex()}
    assert nostr.verify_event(resigned_by_other) != []
    assert nostr.verify_event({"kind": 1}) == ["malformed_event"]
    # unicode content is hashed as UTF-8, not as escapes
    assert nostr.event_id("aa" * 32, 1, 1, [], "naïve") != nostr.event_id("aa" * 32, 1, 1, [], "naive")
