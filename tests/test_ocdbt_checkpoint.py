"""OCDBT key-value databases and the Orbax checkpoint layout built on them: codec round trips, hand-assembled byte
fixtures of each on-disk structure, multi-level and merged multi-process trees, corruption detection, and full
checkpoints written under one mesh and restored under another (``olmax/checkpoint/utils.py:55-221`` and
``olmax/train/checkpointer.py:98-283`` of the reference are the layouts being matched)."""

import json
import struct
from pathlib import Path

import pytest
import torch

from olmax_b200.checkpoint import ocdbt
from olmax_b200.checkpoint import orbax_layout as ol
from olmax_b200.checkpoint.zarr3 import crc32c
from olmax_b200.testing import run_distributed_test


# ----------------------------------------------------------------------------------------------------------------------
# codec
# ----------------------------------------------------------------------------------------------------------------------
def test_varint_round_trip_and_limits():
    for n in (0, 1, 127, 128, 300, 2**32, 2**63 + 5):
        enc = ocdbt.encode_varint(n)
        assert ocdbt.decode_varint(enc + b"\xff", 0) == (n, len(enc))
    assert ocdbt.encode_varint(300) == b"\xac\x02"
    with pytest.raises(ocdbt.OcdbtFormatError):
        ocdbt.decode_varint(b"\x80", 0)
    with pytest.raises(ValueError):
        ocdbt.encode_varint(-1)


def _framed(magic, body):
    head = struct.pack(">I", magic) + struct.pack("<Q", 4 + 8 + 2 + len(body) + 4) + b"\x00\x00" + body
    return head + struct.pack("<I", crc32c(head))


def test_hand_built_leaf_node_parses():
    """A leaf with two keys sharing a prefix: 'ab/x' inline ('hi') and 'ab/y' out of line in file 'p/' + 'd/f' at 10+300."""
    body = bytes([0])                                  # height 0
    body += bytes([1]) + bytes([5]) + bytes([2]) + b"p/d/f"   # file table: 1 file, suffix length 5, base length 2
    body += bytes([2])                                 # two entries
    body += bytes([3])                                 # key 1 shares 3 bytes with key 0
    body += bytes([4, 1]) + b"ab/x" + b"y"             # suffix lengths, suffix bytes
    body += bytes([2]) + b"\xac\x02"                   # value lengths 2, 300
    body += bytes([0, 1])                              # kinds: inline, out of line
    body += bytes([0]) + bytes([10])                   # out-of-line: file index 0, offset 10
    body += b"hi"                                      # inline bytes
    height, entries = ocdbt.decode_node(_framed(ocdbt.MAGIC_BTREE_NODE, body))
    assert height == 0
    (k0, v0), (k1, v1) = entries
    assert (k0, v0.inline) == (b"ab/x", b"hi")
    assert k1 == b"ab/y" and v1.inline is None and (v1.offset, v1.length) == (10, 300)
    assert (v1.file.base_path, v1.file.relative_path) == ("p/", "d/f")
    # the encoder produces the same bytes
    again = ocdbt.encode_leaf([(b"ab/x", ocdbt.ValueRef(b"hi")),
                               (b"ab/y", ocdbt.ValueRef(None, ocdbt.DataFile("p/", "d/f"), 10, 300))])
    assert again == _framed(ocdbt.MAGIC_BTREE_NODE, body)


def test_hand_built_manifest_parses_and_detects_damage():
    body = bytes(range(16))                            # uuid
    body += bytes([0, 100]) + b"\x80\x80\x80\x04" + bytes([4, 0])   # kind, max inline 100, max node 8 MiB, arity 2^4, no compression
    body += bytes([1, 3, 0]) + b"d/a"                  # file table: 'd/a', no base path
    body += bytes([1, 7, 2])                           # one version: generation 7, root height 2
    body += bytes([0, 64]) + b"\x90\x03"               # root: file 0, offset 64, length 400
    body += bytes([5]) + b"\xe8\x07" + b"\xc0\x3e"     # 5 keys, 1000 tree bytes, 8000 indirect bytes
    body += struct.pack("<Q", 1234567)                 # commit time
    body += bytes([0])                                 # no version-tree nodes
    blob = _framed(ocdbt.MAGIC_MANIFEST, body)
    m = ocdbt.decode_manifest(blob)
    v = m.latest
    assert m.uuid == bytes(range(16)) and m.max_inline_value_bytes == 100 and m.max_decoded_node_bytes == 8 << 20
    assert (v.generation, v.root_height, v.root_file.full, v.root_offset, v.root_length) == (7, 2, "d/a", 64, 400)
    assert (v.num_keys, v.tree_bytes, v.indirect_bytes, v.commit_time_ns) == (5, 1000, 8000, 1234567)
    assert ocdbt.encode_manifest(m) == blob
    damaged = bytearray(blob)
    damaged[20] ^= 1
    with pytest.raises(ocdbt.OcdbtFormatError, match="CRC"):
        ocdbt.decode_manifest(bytes(damaged))
    with pytest.raises(ocdbt.OcdbtFormatError, match="magic"):
        ocdbt.decode_node(blob)
    with pytest.raises(ocdbt.OcdbtFormatError, match="length"):
        ocdbt.decode_manifest(blob + b"\x00")


@pytest.mark.parametrize("fanout,compress", [(512, False), (3, False), (4, True)])
def test_database_round_trip_multi_level(tmp_path, fanout, compress):
    if compress and ocdbt._zstd() is None:
        pytest.skip("libzstd not present")
    w = ocdbt.OcdbtWriter(tmp_path / "db", fanout=fanout, compress_nodes=compress)
    want = {}
    for i in range(41):
        key = f"layers.{i % 7}.w{i}/c/{i}"
        val = bytes([i]) * (i * 37 % 500)     # some inline (<= 100 bytes), some out of line, one empty
        w.put(key, val)
        want[key] = val
    big = torch.arange(100000, dtype=torch.float32)
    w.put("big/c/0", memoryview(big.numpy()).cast("B"))
    want["big/c/0"] = big.numpy().tobytes()
    m = w.commit()
    assert m.latest.num_keys == 42 and (m.latest.root_height >= 2) == (fanout < 8)
    with ocdbt.OcdbtReader(tmp_path / "db") as r:
        assert sorted(r.items()) == sorted(want)
        for k, v in want.items():
            assert r.get(k) == v
        assert r.get("big/c/0", 400, 8) == want["big/c/0"][400:408]
        assert r.keys("layers.3.") == sorted(k for k in want if k.startswith("layers.3."))
        with pytest.raises(KeyError):
            r.get("missing")
    assert len(list((tmp_path / "db" / "d").iterdir())) == 1


def test_merge_of_process_databases_references_their_data_files(tmp_path):
    for p in range(3):
        w = ocdbt.OcdbtWriter(tmp_path / f"ocdbt.process_{p}")
        w.put("w/zarr.json", b'{"replicated": true}')            # inline, written by everyone
        w.put(f"w/c/{p}/0", bytes([p + 1]) * 5000)                # out of line
        w.commit()
    ocdbt.OcdbtWriter(tmp_path / "ocdbt.process_3").commit()      # a process with nothing to write
    m = ocdbt.merge_process_databases(tmp_path, [f"ocdbt.process_{p}" for p in range(4)])
    assert m.latest.num_keys == 4
    with ocdbt.OcdbtReader(tmp_path) as r:
        ref = r.items()["w/c/2/0"]
        assert ref.file.base_path == "ocdbt.process_2/" and ref.file.relative_path.startswith("d/")
        assert r.get("w/c/1/0") == b"\x02" * 5000 and r.get("w/zarr.json") == b'{"replicated": true}'
    # an empty database round-trips too
    with ocdbt.OcdbtReader(tmp_path / "ocdbt.process_3") as r:
        assert r.items() == {}


def test_subtree_common_prefix_is_honoured(tmp_path):
    """Interior nodes may strip a prefix shared by every key of a child; a tree written that way reads back whole."""
    d = tmp_path / "db"
    (d / "d").mkdir(parents=True)
    f = ocdbt.DataFile("", "d/x")
    leaf = ocdbt.encode_leaf([(b"1", ocdbt.ValueRef(b"one")), (b"2", ocdbt.ValueRef(b"two"))])   # keys without 'params.'
    interior = ocdbt.encode_interior(1, [ocdbt._Child(b"params.1", 7, f, 0, len(leaf), 2, len(leaf), 0)])
    (d / "d" / "x").write_bytes(leaf + interior)
    v = ocdbt.Version(1, 1, f, len(leaf), len(interior), 2, len(leaf) + len(interior), 0, 1)
    (d / "manifest.ocdbt").write_bytes(ocdbt.encode_manifest(ocdbt.Manifest(b"u" * 16, [v])))
    with ocdbt.OcdbtReader(d) as r:
        assert r.items().keys() == {"params.1", "params.2"} and r.get("params.2") == b"two"


# ----------------------------------------------------------------------------------------------------------------------
# zarr arrays in a database, scan-mode parameters
# ----------------------------------------------------------------------------------------------------------------------
def test_array_regions_fill_values_and_bfloat16(tmp_path):
    w = ol.ItemWriter(tmp_path, 0)
    full = torch.arange(6 * 8, dtype=torch.float32).view(6, 8)
    w.db.put("a/zarr.json", ol.array_metadata((6, 8), (2, 8), torch.float32))
    for i in (0, 2):                                               # chunk 1 (rows 2-3) is absent: fill value
        w.db.put(ol.chunk_key("a", [i, 0]), ol._tensor_bytes(full[2 * i : 2 * i + 2]))
    ol.write_array(w.db, "scalar", torch.tensor(7, dtype=torch.int32))
    ol.write_array(w.db, "h", torch.tensor([1.5, -2.0], dtype=torch.bfloat16))
    w.commit()
    ol.finalize_item(tmp_path, 1, {"a": {"shape": [6, 8], "dtype": "float32"}, "scalar": {"shape": [], "dtype": "int32"}})
    r = ol.ItemReader(tmp_path)
    got = r.read_region("a", [1, 2], [4, 5])
    want = full.clone()
    want[2:4] = 0
    assert torch.equal(got, want[1:5, 2:7])
    assert r.read("scalar").item() == 7 and r.read("scalar").shape == ()
    assert torch.equal(r.read("h"), torch.tensor([1.5, -2.0], dtype=torch.bfloat16))
    meta = json.loads((tmp_path / "_METADATA").read_text())
    assert meta["use_zarr3"] is True and "('a',)" in meta["tree_metadata"]
    assert meta["tree_metadata"]["('scalar',)"]["key_metadata"] == [{"key": "scalar", "key_type": 2}]
    with pytest.raises(ValueError, match="outside"):
        r.read_region("a", [5, 0], [2, 8])
    r.close()


def _ckpt_worker(path, kind, mode, seed):
    """mode 'save': train two steps, save through the Trainer's checkpointer; 'load': restore into a differently
    initialised model / optimizer and return the logical tensors."""
    import torch

    from olmax_b200.models import TransformerRecipeType
    from olmax_b200.optim import AdamWConfig, ConstantSchedule
    from olmax_b200.parallel import MeshResource, dist_utils
    from olmax_b200.train.checkpointer import SimpleCheckpointer, TrainState

    world = dist_utils.get_world_size()
    res = {"fsdp": lambda: MeshResource.FSDP(world), "hsdp": lambda: MeshResource.HSDP(2, world, 2),
           "tp": lambda: MeshResource.FSDP_with_TP(2, world)}[kind]()
    cfg = TransformerRecipeType("tiny_llama").build_recipe().model
    model = cfg.build(seed=seed, mesh_resource=res, device=torch.device("cpu"))
    optim = AdamWConfig(lr=ConstantSchedule(1e-2), max_grad_norm=1.0).build(model, 2)
    ck = SimpleCheckpointer()
    state = TrainState(step=0, epoch=1, global_train_tokens_seen=0, model=model, optim=optim)
    if mode == "save":
        g = torch.Generator().manual_seed(3)
        for step in range(2):
            for _ in range(2):
                ids = torch.randint(0, 1024, (4, 32), generator=g)
                mine = ids.chunk(model.mesh.data_parallel_size)[model.mesh.data_parallel_rank]
                loss, _ = model(mine, torch.roll(mine, -1, 1))
                loss.backward()
                optim.accumulate()
            optim.step()
        state.step, state.global_train_tokens_seen = 2, 512
        state.data_loader_state = {"batches_processed": 2}
        ck.save(path, state)
    else:
        state = ck.load(path, state)
        assert (state.step, state.epoch, state.global_train_tokens_seen) == (2, 1, 512)
        assert state.data_loader_state == {"batches_processed": 2} and optim.count == 2 and optim.mini_step == 0
    store = model.store
    out = {n: store.full_parameter(n) for n, _ in store.named_parameters()}
    out.update({f"mu.{n}": store.full_tensor_like(n, optim.exp_avg) for n, _ in store.named_parameters()})
    out.update({f"nu.{n}": store.full_tensor_like(n, optim.exp_avg_sq) for n, _ in store.named_parameters()})
    return out


@pytest.mark.parametrize("save_kind,save_world,load_kind,load_world", [("fsdp", 2, "hsdp", 4), ("tp", 4, "fsdp", 1)])
def test_orbax_layout_checkpoint_restores_under_another_mesh(tmp_path, save_kind, save_world, load_kind, load_world):
    path = str(tmp_path / "step2")
    saved = run_distributed_test(_ckpt_worker, world_size=save_world, func_args=(path, save_kind, "save", 1))
    loaded = run_distributed_test(_ckpt_worker, world_size=load_world, func_args=(path, load_kind, "load", 99))
    for rank_state in loaded:
        for name, want in saved[0].items():
            assert torch.equal(rank_state[name], want), name
    # the files and names Orbax would have produced for the reference's TrainState
    root = Path(path)
    top = json.loads((root / "_CHECKPOINT_METADATA").read_text())
    assert set(top["item_handlers"]) == {"params", "static", "opt_state", "trainer"}
    assert json.loads((root / "trainer" / "metadata").read_text())["step"] == 2
    for item in ("params", "opt_state", "static"):
        assert (root / item / "manifest.ocdbt").exists() and (root / item / "_METADATA").exists()
        assert sorted(p.name for p in (root / item).glob("ocdbt.process_*")) == [f"ocdbt.process_{i}" for i in range(save_world)]
    assert (root / "params" / "_sharding").exists()
    r = ol.ItemReader(root / "opt_state")
    names = set(r.array_names())
    # MultiSteps(chain(clip, inject_hyperparams(adamw))): the optax nesting of a clipped, 2-micro-batch run
    assert {"mini_step", "gradient_step", "inner_opt_state.1.count", "inner_opt_state.1.hyperparams.learning_rate",
            "inner_opt_state.1.inner_state.0.count", "inner_opt_state.1.inner_state.0.mu.embedding.weight",
            "inner_opt_state.1.inner_state.0.nu.layers.1.mlp.down_proj.weight", "acc_grads.norm.weight"} <= names
    assert r.read("gradient_step").item() == 2 and r.read("gradient_step").dtype == torch.int32
    assert not r.read("acc_grads.norm.weight").any()          # metadata only: every chunk is the fill value
    assert r.meta("inner_opt_state.1.inner_state.0.mu.embedding.weight")["shape"] == [1024, 256]
    r.close()
    pm = json.loads((root / "params" / "_METADATA").read_text())["tree_metadata"]
    assert pm["('layers', '0', 'attention', 'q_proj', 'weight')"]["key_metadata"][1] == {"key": "0", "key_type": 1}


def test_scan_mode_parameters_load_layer_by_layer(tmp_path):
    """A checkpoint whose layers are stacked as ``layers.0.*`` with a leading [num_layers] dimension (what the reference
    writes with ``scan_layers=True``) restores into per-layer parameters."""
    from olmax_b200.models import TransformerRecipeType
    from olmax_b200.parallel import MeshResource

    cfg = TransformerRecipeType("tiny_llama").build_recipe().model
    src = cfg.build(seed=1, mesh_resource=MeshResource.FSDP(1), device=torch.device("cpu"))
    w = ol.ItemWriter(tmp_path / "params", 0)
    full = {n: src.store.full_parameter(n) for n, _ in src.store.named_parameters()}
    for n, t in full.items():
        parts = n.split(".")
        if parts[0] != "layers":
            ol.write_array(w.db, n, t)
        elif parts[1] == "0":
            stacked = torch.stack([full[".".join(["layers", str(i)] + parts[2:])] for i in range(cfg.num_layers)])
            ol.write_array(w.db, n, stacked)
    w.commit()
    ol.finalize_item(tmp_path / "params", 1, {})
    dst = cfg.build(seed=2, mesh_resource=MeshResource.FSDP(1), device=torch.device("cpu"))
    ol.restore_store_item(tmp_path / "params", dst.store, {"": dst.store.master})
    for n in full:
        assert torch.equal(dst.store.full_parameter(n), full[n]), n
