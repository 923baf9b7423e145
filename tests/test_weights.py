"""The MoE weight path on the host (r-mda_b200/host/moe_weights.c): safetensors shards ->
staging bank, against files written here with numpy.  The layout checked is the reference's
(mda_qwen_put_moe, src/qwen.c:441-452): router rows, shared gate row, zero rows up to E + 128,
shared gate_proj, up_proj, down_proj in the dense stage; the fused expert tensors in their own."""
import ctypes as C
import json
import struct

import numpy as np
import pytest

PREFIX = "model.language_model."   # MDA_QWEN_PREFIX, src/qwen.h:12


class Stage(C.Structure):
    _fields_ = [("host", C.c_void_p), ("size", C.c_uint64), ("used", C.c_uint64)]


class Bank(C.Structure):
    _fields_ = [("dense", Stage), ("gu", Stage), ("down", Stage), ("moe", C.c_uint64), ("sdown", C.c_uint64),
                ("pinned", C.c_bool), ("fail", C.c_bool), ("c", C.c_void_p)]


class BankCfg(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("d", "experts", "inter", "shared")]


class StSet(C.Structure):
    _fields_ = [("files", C.c_void_p), ("n", C.c_uint32)]


class StTensor(C.Structure):
    _fields_ = [("data", C.c_void_p), ("rows", C.c_uint64), ("cols", C.c_uint32), ("dtype", C.c_uint32), ("ok", C.c_bool)]


class BankJob(C.Structure):
    _fields_ = [("b", C.POINTER(Bank)), ("set", C.POINTER(StSet)), ("prefix", C.c_char_p), ("cfg", BankCfg),
                ("layer", C.c_uint32), ("th", C.c_ulong), ("started", C.c_bool), ("e_lo", C.c_uint32), ("e_hi", C.c_uint32)]


@pytest.fixture(scope="module")
def wlib(pkg):
    pkg.build.build_host()
    L = C.CDLL(pkg.build.HOST_LIB)
    L.moe_st_open_set.restype = StSet
    L.moe_st_open_set.argtypes = [C.c_char_p]
    L.moe_st_free_set.argtypes = [C.POINTER(StSet)]
    L.moe_st_find.restype = StTensor
    L.moe_st_find.argtypes = [C.POINTER(StSet), C.c_char_p]
    L.moe_st_bf16.restype = C.c_float
    L.moe_st_bf16.argtypes = [C.c_void_p, C.c_uint64]
    L.moe_bank_open.restype = C.c_bool
    L.moe_bank_open.argtypes = [C.POINTER(Bank), C.c_void_p, BankCfg]
    L.moe_bank_close.argtypes = [C.POINTER(Bank)]
    L.moe_bank_reset.argtypes = [C.POINTER(Bank)]
    L.moe_bank_put_moe.argtypes = [C.POINTER(Bank), C.POINTER(StSet), C.c_char_p, BankCfg, C.c_uint32]
    L.moe_bank_open_slice.restype = C.c_bool
    L.moe_bank_open_slice.argtypes = [C.POINTER(Bank), C.c_void_p, BankCfg, C.c_uint32]
    L.moe_bank_put_moe_slice.argtypes = [C.POINTER(Bank), C.POINTER(StSet), C.c_char_p, BankCfg, C.c_uint32, C.c_uint32, C.c_uint32]
    L.moe_bank_upload.argtypes = [C.POINTER(Bank), C.c_void_p, C.c_void_p, C.c_void_p, C.c_bool]
    L.moe_bank_prefetch.argtypes = [C.POINTER(BankJob)]
    L.moe_bank_join.argtypes = [C.POINTER(BankJob)]
    return L


def write_safetensors(path, tensors, pretty=False, metadata=None):
    """tensors: name -> (dtype string, uint16/int64 array).  Offsets in file order."""
    header, blobs, at = {}, [], 0
    if metadata is not None:
        header["__metadata__"] = metadata
    for name, (dt, a) in tensors.items():
        raw = np.ascontiguousarray(a).tobytes()
        header[name] = {"dtype": dt, "shape": list(a.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    text = json.dumps(header, indent=2) if pretty else json.dumps(header, separators=(",", ":"))
    text += " " * (-len(text) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text.encode())
        for b in blobs:
            f.write(b)


def layer_tensors(rng, l, d, E, I, S):
    def bf(*shape):
        return rng.integers(0, 1 << 16, shape).astype(np.uint16)
    base = f"{PREFIX}layers.{l}.mlp."
    t = {base + "gate.weight": ("BF16", bf(E, d)),
         base + "experts.gate_up_proj": ("BF16", bf(E, 2 * I, d)),
         base + "experts.down_proj": ("BF16", bf(E, d, I))}
    if S:
        t.update({base + "shared_expert_gate.weight": ("BF16", bf(1, d)),
                  base + "shared_expert.gate_proj.weight": ("BF16", bf(S, d)),
                  base + "shared_expert.up_proj.weight": ("BF16", bf(S, d)),
                  base + "shared_expert.down_proj.weight": ("BF16", bf(d, S))})
    return t


def stage_bytes(st):
    return np.frombuffer(C.string_at(st.host, st.used), np.uint16) if st.used else np.zeros(0, np.uint16)


def expected_dense(t, l, d, E, S):
    base = f"{PREFIX}layers.{l}.mlp."
    rows = [t[base + "gate.weight"][1]]
    if S:
        rows.append(t[base + "shared_expert_gate.weight"][1])
    n = sum(r.shape[0] for r in rows)
    rows.append(np.zeros((E + 128 - n, d), np.uint16))
    if S:
        rows += [t[base + "shared_expert.gate_proj.weight"][1], t[base + "shared_expert.up_proj.weight"][1]]
    flat = np.concatenate([r.ravel() for r in rows])
    if S:
        flat = np.concatenate([flat, t[base + "shared_expert.down_proj.weight"][1].ravel()])
    return flat


@pytest.mark.parametrize("S", [0, 64])
def test_expert_slice_staging(wlib, tmp_path, S):
    """Expert parallel: every rank stages the replicated dense block whole and only its own experts' rows of the
    two fused expert tensors; the slices of all ranks put together are the full tensors."""
    d, E, I, G = 64, 8, 32, 4
    rng = np.random.default_rng(5)
    l0 = layer_tensors(rng, 0, d, E, I, S)
    write_safetensors(tmp_path / "model.safetensors", l0)
    st = wlib.moe_st_open_set(str(tmp_path).encode())
    cfg = BankCfg(d, E, I, S)
    base = f"{PREFIX}layers.0.mlp."
    gu_full, down_full = l0[base + "experts.gate_up_proj"][1], l0[base + "experts.down_proj"][1]
    got_gu, got_down = [], []
    el = E // G
    for g in range(G):
        bank = Bank()
        assert wlib.moe_bank_open_slice(C.byref(bank), None, cfg, el)
        assert bank.gu.size == el * 2 * I * d * 2 and bank.down.size == el * d * I * 2
        if g % 2 == 0:
            wlib.moe_bank_put_moe_slice(C.byref(bank), C.byref(st), PREFIX.encode(), cfg, 0, g * el, (g + 1) * el)
        else:   # the loader thread takes the same slice
            job = BankJob(C.pointer(bank), C.pointer(st), PREFIX.encode(), cfg, 0, 0, False, g * el, (g + 1) * el)
            wlib.moe_bank_prefetch(C.byref(job))
            wlib.moe_bank_join(C.byref(job))
        assert not bank.fail
        assert np.array_equal(stage_bytes(bank.dense), expected_dense(l0, 0, d, E, S))
        got_gu.append(stage_bytes(bank.gu).copy())
        got_down.append(stage_bytes(bank.down).copy())
        wlib.moe_bank_close(C.byref(bank))
    assert np.array_equal(np.concatenate(got_gu), gu_full.ravel())
    assert np.array_equal(np.concatenate(got_down), down_full.ravel())
    bank = Bank()
    assert wlib.moe_bank_open_slice(C.byref(bank), None, cfg, el)
    wlib.moe_bank_put_moe_slice(C.byref(bank), C.byref(st), PREFIX.encode(), cfg, 0, 6, 9)     # beyond the last expert
    assert bank.fail
    wlib.moe_bank_reset(C.byref(bank))
    wlib.moe_bank_put_moe_slice(C.byref(bank), C.byref(st), PREFIX.encode(), cfg, 0, 0, 3)     # more experts than the stages hold
    assert bank.fail
    wlib.moe_bank_close(C.byref(bank))
    wlib.moe_st_free_set(C.byref(st))


@pytest.mark.parametrize("S", [0, 64])
def test_shards_to_bank(wlib, tmp_path, S):
    d, E, I = 64, 8, 32
    rng = np.random.default_rng(3)
    l0, l1 = layer_tensors(rng, 0, d, E, I, S), layer_tensors(rng, 1, d, E, I, S)
    # two shards, tensors of a layer split across them, one compact header and one indented with metadata
    names0 = list(l0)
    write_safetensors(tmp_path / "model-00001-of-00002.safetensors",
                      {**{k: l0[k] for k in names0[:2]}, **l1, "ids": ("I64", np.arange(5, dtype=np.int64))})
    write_safetensors(tmp_path / "model-00002-of-00002.safetensors", {k: l0[k] for k in names0[2:]}, pretty=True,
                      metadata={"format": "pt", "note": 'a "quoted" {brace} in a string'})
    (tmp_path / "config.json").write_text("{}")
    st = wlib.moe_st_open_set(str(tmp_path).encode())
    assert st.n == 2
    t = wlib.moe_st_find(C.byref(st), (PREFIX + "layers.1.mlp.experts.down_proj").encode())
    assert t.ok and (t.rows, t.cols, t.dtype) == (E * d, I, 0)       # leading dimensions fold into rows
    assert wlib.moe_st_find(C.byref(st), b"ids").dtype == 1 and not wlib.moe_st_find(C.byref(st), b"absent").ok
    one = np.array([0x3FC0], np.uint16)                                # 1.5 in bf16
    assert wlib.moe_st_bf16(one.ctypes.data, 0) == 1.5
    cfg = BankCfg(d, E, I, S)
    bank = Bank()
    assert wlib.moe_bank_open(C.byref(bank), None, cfg)
    for l, tens in ((0, l0), (1, l1), (0, l0)):                        # a bank is reused layer after layer
        wlib.moe_bank_reset(C.byref(bank))
        wlib.moe_bank_put_moe(C.byref(bank), C.byref(st), PREFIX.encode(), cfg, l)
        assert not bank.fail
        base = f"{PREFIX}layers.{l}.mlp."
        assert np.array_equal(stage_bytes(bank.dense), expected_dense(tens, l, d, E, S))
        assert np.array_equal(stage_bytes(bank.gu), tens[base + "experts.gate_up_proj"][1].ravel())
        assert np.array_equal(stage_bytes(bank.down), tens[base + "experts.down_proj"][1].ravel())
        assert bank.moe == 0 and bank.sdown == ((E + 128 + 2 * S) * d if S else 0)
    # the loader thread gives the same bank contents
    job = BankJob(C.pointer(bank), C.pointer(st), PREFIX.encode(), cfg, 1, 0, False, 0, 0)
    wlib.moe_bank_prefetch(C.byref(job))
    wlib.moe_bank_join(C.byref(job))
    assert not bank.fail and np.array_equal(stage_bytes(bank.gu), l1[f"{PREFIX}layers.1.mlp.experts.gate_up_proj"][1].ravel())
    # a layer that is not there, and a shape that does not match the configuration
    wlib.moe_bank_reset(C.byref(bank))
    wlib.moe_bank_put_moe(C.byref(bank), C.byref(st), PREFIX.encode(), cfg, 2)
    assert bank.fail
    wlib.moe_bank_reset(C.byref(bank))
    wlib.moe_bank_put_moe(C.byref(bank), C.byref(st), PREFIX.encode(), BankCfg(d, E, 2 * I, S), 0)
    assert bank.fail
    wlib.moe_bank_close(C.byref(bank))
    wlib.moe_st_free_set(C.byref(st))


def test_damaged_shards_are_refused(wlib, tmp_path):
    rng = np.random.default_rng(4)
    good = layer_tensors(rng, 0, 32, 4, 32, 0)
    write_safetensors(tmp_path / "a.safetensors", good)
    raw = (tmp_path / "a.safetensors").read_bytes()
    cases = {
        "short": raw[:len(raw) - 10],                                  # data_offsets run past the end of the file
        "hlen": struct.pack("<Q", 1 << 40) + raw[8:],                  # header length larger than the file
        "json": raw[:8] + raw[8:].replace(b'"shape"', b'"shaqe"', 1),  # an entry without a shape
    }
    for name, blob in cases.items():
        sub = tmp_path / name
        sub.mkdir()
        (sub / "a.safetensors").write_bytes(blob)
        st = wlib.moe_st_open_set(str(sub).encode())
        if st.n != 0:                                                   # the file maps, the tensor must not resolve
            key = (PREFIX + "layers.0.mlp.experts.down_proj").encode()
            assert not wlib.moe_st_find(C.byref(st), key).ok, name
            wlib.moe_st_free_set(C.byref(st))
    empty = tmp_path / "empty"
    empty.mkdir()
    assert wlib.moe_st_open_set(str(empty).encode()).n == 0
    assert wlib.moe_st_open_set(str(tmp_path / "nowhere").encode()).n == 0


def test_header_scanner_survives_mutations(wlib, tmp_path):
    """Seeded byte mutations, insertions, deletions and truncations of a valid shard: the reader either
    refuses the file or hands out tensors whose bytes lie inside the mapping."""
    import random
    rng = np.random.default_rng(6)
    write_safetensors(tmp_path / "a.safetensors", layer_tensors(rng, 0, 32, 4, 32, 32), pretty=True, metadata={"k": "v"})
    raw = (tmp_path / "a.safetensors").read_bytes()
    hlen = struct.unpack("<Q", raw[:8])[0]
    names = [(PREFIX + "layers.0.mlp." + n).encode() for n in ("gate.weight", "experts.gate_up_proj", "experts.down_proj")]
    random.seed(1)
    sub = tmp_path / "m"
    sub.mkdir()
    parsed = 0
    for _ in range(400):
        b = bytearray(raw)
        for _ in range(random.randint(1, 4)):
            pos, mode = random.randint(0, 8 + hlen - 1), random.random()
            if mode < 0.5:
                b[pos] = random.randint(0, 255)
            elif mode < 0.7:
                b[pos] = random.choice(b'{}[]",:\\ 0123456789')
            elif mode < 0.85:
                del b[pos]
            else:
                b.insert(pos, random.choice(b'{}[]",:\\ 9'))
        if random.random() < 0.2:
            b = b[:random.randint(0, len(b))]
        (sub / "x.safetensors").write_bytes(bytes(b))
        st = wlib.moe_st_open_set(str(sub).encode())
        if st.n:
            parsed += 1
            for nm in names:
                t = wlib.moe_st_find(C.byref(st), nm)
                if t.ok:                                                    # first and last byte must be readable
                    C.string_at(t.data, 1)
                    C.string_at(t.data + t.rows * t.cols * 2 - 1, 1)
            wlib.moe_st_free_set(C.byref(st))
    assert 0 < parsed < 400


@pytest.mark.gpu
def test_bank_upload_converts_in_place(wlib, ctx, oracle, tmp_path):
    """Shards -> page-locked bank -> device, bf16 rewritten as fp16 (mda_qwen_upload, src/qwen.c:381-394)."""
    d, E, I, S = 128, 8, 64, 64
    rng = np.random.default_rng(5)
    tens = layer_tensors(rng, 0, d, E, I, S)
    for k, (dt, a) in tens.items():                                    # finite values only: NaN payloads need not survive
        a[(a & 0x7F80) == 0x7F80] &= 0x3FFF
    write_safetensors(tmp_path / "m.safetensors", tens)
    st = wlib.moe_st_open_set(str(tmp_path).encode())
    cfg = BankCfg(d, E, I, S)
    bank = Bank()
    assert wlib.moe_bank_open(C.byref(bank), ctx.p, cfg)
    wlib.moe_bank_put_moe(C.byref(bank), C.byref(st), PREFIX.encode(), cfg, 0)
    assert not bank.fail
    host = {n: stage_bytes(getattr(bank, n)).copy() for n in ("dense", "gu", "down")}
    dev = {n: ctx.alloc(getattr(bank, n).size) for n in host}
    wlib.moe_bank_upload(C.byref(bank), dev["dense"].ptr, dev["gu"].ptr, dev["down"].ptr, True)
    ctx.flush()
    for n, h in host.items():
        got = dev[n].read(np.uint32, (h.size // 2,))
        assert np.array_equal(got, oracle.bf16_to_f16(np.ascontiguousarray(h.view(np.uint32)))), n
    wlib.moe_bank_close(C.byref(bank))
    wlib.moe_st_free_set(C.byref(st))
