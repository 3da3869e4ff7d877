"""Data-loading modules: OFRecord codec against protobuf's wire format, readers, decoders, image ops
(CPU; reference behaviour: python/oneflow/nn/modules/dataset.py, oneflow/user/data/*)."""
import io
import json
import os

import numpy as np
import pytest
import torch

import oneflow as flow
from oneflow_b200.nn.modules.dataset import MegatronIndexedDataset
from oneflow_b200.utils import ofrecord as rec


def _png(h, w, seed):
    from PIL import Image
    a = (np.random.RandomState(seed).rand(h, w, 3) * 255).astype(np.uint8)
    b = io.BytesIO()
    Image.fromarray(a).save(b, format="PNG")
    return b.getvalue(), a


@pytest.fixture(scope="module")
def dataset(tmp_path_factory):
    d = str(tmp_path_factory.mktemp("ofrecord"))
    imgs = {}
    for part in range(4):
        recs = []
        for i in range(10):
            k = part * 10 + i
            by, a = _png(40 + k % 3, 50 + k % 5, k)
            imgs[k] = a
            recs.append({"encoded": by, "class/label": np.array([k], np.int32), "vec": np.arange(6, dtype=np.float32) + k,
                         "ids": np.arange(k % 4 + 1, dtype=np.int64)})
        rec.write_ofrecord_file(f"{d}/part-{part}", recs)
    return d, imgs


def test_codec_matches_protobuf_wire_format():
    from google.protobuf import descriptor_pb2, descriptor_pool, message_factory
    F = descriptor_pb2.FieldDescriptorProto
    fd = descriptor_pb2.FileDescriptorProto(name="rec.proto", package="t", syntax="proto2")
    for name, typ, packed in (("BytesList", F.TYPE_BYTES, False), ("FloatList", F.TYPE_FLOAT, True), ("DoubleList", F.TYPE_DOUBLE, True),
                              ("Int32List", F.TYPE_INT32, True), ("Int64List", F.TYPE_INT64, True)):
        m = fd.message_type.add(name=name)
        f = m.field.add(name="value", number=1, type=typ, label=3)
        if packed:
            f.options.packed = True
    feat = fd.message_type.add(name="Feature")
    feat.oneof_decl.add(name="kind")
    for i, (n, t) in enumerate((("bytes_list", "BytesList"), ("float_list", "FloatList"), ("double_list", "DoubleList"),
                                ("int32_list", "Int32List"), ("int64_list", "Int64List")), 1):
        feat.field.add(name=n, number=i, type=F.TYPE_MESSAGE, type_name=".t." + t, label=1, oneof_index=0)
    r = fd.message_type.add(name="OFRecord")
    ent = r.nested_type.add(name="FeatureEntry")
    ent.options.map_entry = True
    ent.field.add(name="key", number=1, type=F.TYPE_STRING, label=1)
    ent.field.add(name="value", number=2, type=F.TYPE_MESSAGE, type_name=".t.Feature", label=1)
    r.field.add(name="feature", number=1, type=F.TYPE_MESSAGE, type_name=".t.OFRecord.FeatureEntry", label=3)
    pool = descriptor_pool.DescriptorPool()
    pool.Add(fd)
    OFRecord = message_factory.GetMessageClass(pool.FindMessageTypeByName("t.OFRecord"))

    msg = OFRecord()
    msg.feature["img"].bytes_list.value.append(b"\x00\x01\xff" * 10)
    msg.feature["f"].float_list.value.extend([1.5, -2.25, 3e8])
    msg.feature["d"].double_list.value.extend([1e-300, 2.0])
    msg.feature["i"].int32_list.value.extend([-1, 0, 5, 2 ** 31 - 1, -2 ** 31])
    msg.feature["l"].int64_list.value.extend([-1, 2 ** 62, -2 ** 63, 7])
    blob = msg.SerializeToString()
    d = rec.decode_ofrecord(blob)
    assert d["img"][1] == [b"\x00\x01\xff" * 10]
    assert np.allclose(d["f"][1], [1.5, -2.25, 3e8]) and list(d["d"][1]) == [1e-300, 2.0]
    assert list(d["i"][1]) == [-1, 0, 5, 2 ** 31 - 1, -2 ** 31]
    assert list(d["l"][1]) == [-1, 2 ** 62, -2 ** 63, 7]
    assert rec.decode_feature(blob, "i")[0] == "int32"
    with pytest.raises(KeyError):
        rec.decode_feature(blob, "missing")

    mine = rec.encode_ofrecord({"img": b"abc", "f": np.array([1., 2.], np.float32), "i": np.array([-3, 4], np.int32),
                                "l": np.array([-5, 2 ** 40]), "d": np.array([.5])})
    back = OFRecord()
    back.ParseFromString(mine)
    assert back.feature["img"].bytes_list.value[0] == b"abc"
    assert list(back.feature["i"].int32_list.value) == [-3, 4] and list(back.feature["l"].int64_list.value) == [-5, 2 ** 40]
    assert list(back.feature["f"].float_list.value) == [1., 2.] and list(back.feature["d"].double_list.value) == [.5]


def test_ofrecord_reader_and_decoders(dataset):
    d, imgs = dataset
    r = flow.nn.OFRecordReader(d, batch_size=8, data_part_num=4, random_shuffle=False)
    lab = flow.nn.OFRecordRawDecoder("class/label", shape=(), dtype=flow.int32)
    vec = flow.nn.OFRecordRawDecoder("vec", shape=(2, 3), dtype=flow.float32)
    ids = flow.nn.OFRecordRawDecoder("ids", shape=(4,), dtype=flow.int64, dim1_varying_length=True)
    dec = flow.nn.OFRecordImageDecoder("encoded", color_space="RGB")
    seen = []
    for _ in range(10):
        b = r()
        la = lab(b)
        seen += la.tolist()
        v = vec(b)
        assert v.shape == (8, 2, 3) and torch.equal(v[:, 0, 0], la.float())
        assert ids(b).shape == (8, 4)
        for t, k in zip(dec(b).tensors, la.tolist()):
            assert np.array_equal(t.numpy(), imgs[k])
    assert seen[:40] == list(range(40)) and seen[40:80] == list(range(40))      # epochs roll over in order
    with pytest.raises(ValueError):
        flow.nn.OFRecordRawDecoder("vec", shape=(2,), dtype=flow.float32)(b)    # longer than shape, no truncate
    assert flow.nn.OFRecordRawDecoder("vec", shape=(2,), dtype=flow.float32, truncate=True)(b).shape == (8, 2)
    bgr = flow.nn.OFRecordImageDecoder("encoded", color_space="BGR")(b).tensors[0]
    assert torch.equal(bgr.flip(2), dec(b).tensors[0])


def test_ofrecord_reader_shuffles_without_losing_records(dataset):
    d, _ = dataset
    r = flow.nn.OfrecordReader(d, batch_size=10, data_part_num=4, random_shuffle=True, shuffle_after_epoch=True, random_seed=3,
                               shuffle_buffer_size=16)
    lab = flow.nn.OfrecordRawDecoder("class/label", shape=(), dtype=flow.int32)
    e = []
    for _ in range(4):
        e += lab(r()).tolist()
    assert sorted(e) == list(range(40)) and e != list(range(40))


def test_image_pipeline(dataset):
    d, imgs = dataset
    r = flow.nn.OFRecordReader(d, batch_size=8, data_part_num=4)
    b = r()
    lab = flow.nn.OFRecordRawDecoder("class/label", shape=(), dtype=flow.int32)(b)
    crops = flow.nn.OFRecordImageDecoderRandomCrop("encoded", color_space="BGR", random_seed=1)(b)
    dense, scale, _ = flow.nn.image.Resize(target_size=(32, 24))(crops)
    assert dense.shape == (8, 24, 32, 3) and dense.dtype == torch.uint8 and scale.shape == (8, 2)
    flip = flow.nn.CoinFlip(batch_size=8, random_seed=5)()
    assert flip.dtype == torch.int8 and flip.shape == (8,)
    cmn = flow.nn.CropMirrorNormalize(crop_h=20, crop_w=28, mean=[1., 2., 3.], std=[2., 2., 2.])
    y = cmn(dense, flip)
    ref = (dense[:, 2:22, 2:30].float() - torch.tensor([1., 2., 3.])) / 2
    ref = torch.where(flip.bool().view(-1, 1, 1, 1), ref.flip(2), ref).permute(0, 3, 1, 2)
    assert y.shape == (8, 3, 20, 28) and torch.allclose(y, ref)

    full = flow.nn.OFRecordImageDecoder("encoded", color_space="RGB")(b)
    o, sc, sz = flow.nn.image.Resize(target_size=20, keep_aspect_ratio=True, max_size=24)(full)
    assert all(min(t.shape[:2]) <= 20 and max(t.shape[:2]) <= 24 for t in o.tensors)
    assert sz.tolist() == [[t.shape[1], t.shape[0]] for t in o.tensors]
    al = flow.nn.image.batch_align(shape=(0, 0, 3), dtype=flow.float32, alignment=16)(o)
    assert al.shape[1] % 16 == 0 and al.shape[2] % 16 == 0 and torch.equal(al[0, :o.tensors[0].shape[0], :o.tensors[0].shape[1]], o.tensors[0].float())
    fl = flow.nn.image.flip()(o, torch.tensor([1, 2, 3, 0, 1, 1, 1, 1]))
    assert torch.equal(fl.tensors[0], o.tensors[0].flip(1)) and torch.equal(fl.tensors[1], o.tensors[1].flip(0))
    assert torch.equal(fl.tensors[2], o.tensors[2].flip(0, 1)) and torch.equal(fl.tensors[3], o.tensors[3])
    nm = flow.nn.image.normalize([2., 2., 2.], [1., 1., 1.])(o)
    assert torch.allclose(nm.tensors[0], (o.tensors[0].float() - 1) / 2)

    raw = flow.nn.OFRecordBytesDecoder("encoded")(b)
    g = flow.nn.OFRecordImageGpuDecoderRandomCropResize(16, 12, seed=1)(raw)
    assert g.shape == (8, 12, 16, 3) and g.dtype == torch.uint8
    di = flow.nn.image.decode(color_space="RGB")(raw)
    assert np.array_equal(di.tensors[0].numpy(), imgs[lab[0].item()])


def test_raw_reader(tmp_path):
    raw = np.arange(100 * 6, dtype=np.float32).reshape(100, 6)
    raw[:50].tofile(tmp_path / "r0.bin")
    raw[50:].tofile(tmp_path / "r1.bin")
    files = [str(tmp_path / "r0.bin"), str(tmp_path / "r1.bin")]
    rr = flow.nn.RawReader(files, shape=(2, 3), dtype=flow.float32, batch_size=10, random_shuffle=False)
    x = rr()
    assert x.shape == (10, 2, 3) and torch.equal(x.reshape(10, 6), torch.from_numpy(raw[:10]))
    for _ in range(5):
        x = rr()
    assert torch.equal(x.reshape(10, 6), torch.from_numpy(raw[50:60]))          # crossed into the second file
    rs = flow.nn.RawReader(files, shape=(6,), dtype=flow.float32, batch_size=10, random_shuffle=True, shuffle_block_size=5, random_seed=1)
    al = torch.cat([rs() for _ in range(10)])
    assert sorted(al[:, 0].tolist()) == list(raw[:, 0]) and al[:, 0].tolist() != list(raw[:, 0])
    assert torch.equal(al[:5, 0] - al[0, 0], torch.arange(5.) * 6)              # blocks stay contiguous


def test_gpt_indexed_reader(tmp_path):
    rng = np.random.RandomState(0)
    docs = [rng.randint(0, 1000, size=n).astype(np.uint16) for n in rng.randint(5, 40, size=30)]
    prefix = str(tmp_path / "gpt")
    MegatronIndexedDataset.write(prefix, docs)
    stream = np.concatenate(docs)
    gr = flow.nn.GPTIndexedBinDataReader(prefix, seq_length=16, num_samples=20, batch_size=4, shuffle=False)
    o = gr()
    assert o.shape == (4, 17) and o.dtype == torch.int64
    for b in range(4):                                                           # one token of overlap between samples
        assert np.array_equal(o[b].numpy(), stream[16 * b:16 * b + 17])
    gs = flow.nn.GPTIndexedBinDataReader(prefix, seq_length=16, num_samples=200, batch_size=4, shuffle=True, random_seed=2,
                                         split_sizes=(8, 2), split_index=0)
    first = [gs() for _ in range(3)]
    assert all(t.shape == (4, 17) for t in first)
    again = flow.nn.GPTIndexedBinDataReader(prefix, seq_length=16, num_samples=200, batch_size=4, shuffle=True, random_seed=2,
                                            split_sizes=(8, 2), split_index=0)
    assert torch.equal(again(), first[0])                                        # seeded: reproducible
    with pytest.raises(ValueError):
        flow.nn.GPTIndexedBinDataReader(prefix, seq_length=16, num_samples=20, batch_size=4, split_sizes=(1,), split_index=1)


def test_coco_reader(tmp_path):
    os.makedirs(tmp_path / "img")
    ims, ann = [], []
    for i in range(6):
        by, _ = _png(30 + 10 * (i % 2), 40, i)
        (tmp_path / "img" / f"{i}.png").write_bytes(by)
        ims.append({"id": i + 100, "file_name": f"{i}.png", "height": 30 + 10 * (i % 2), "width": 40})
        ann.append({"id": i, "image_id": i + 100, "bbox": [5, 5, 10, 12], "category_id": 7 if i % 2 else 3, "iscrowd": 0,
                    "segmentation": [[1, 1, 5, 1, 5, 5, 1, 5]]})
    ann.append({"id": 99, "image_id": 100, "bbox": [0, 0, 50, 50], "category_id": 3, "iscrowd": 1, "segmentation": []})
    ims.append({"id": 999, "file_name": "none.png", "height": 10, "width": 10})       # no annotations: dropped
    (tmp_path / "a.json").write_text(json.dumps({"images": ims, "annotations": ann, "categories": [{"id": 7}, {"id": 3}]}))
    cr = flow.nn.COCOReader(str(tmp_path / "a.json"), str(tmp_path / "img"), batch_size=2, shuffle=True, random_seed=0)
    seen = set()
    for _ in range(6):
        image, iid, isz, bb, lb, sg, sgi = cr()
        assert len(image) == 2 and iid.shape == (2,) and isz.shape == (2, 2)
        seen.update(iid.tolist())
        for k in range(2):
            assert bb.tensors[k].tolist() == [[5, 5, 14, 16]]                       # xyxy = (l, t, l + w - 1, t + h - 1)
            assert lb.tensors[k].item() == (2 if (iid[k].item() - 100) % 2 else 1)  # contiguous ids by ascending category id
            assert sg.tensors[k].shape == (4, 2) and sgi.tensors[k][:, 0].tolist() == [0, 1, 2, 3]
    assert seen == {100, 101, 102, 103, 104, 105}
