"""Dataset plumbing on synthetic files: readers, event->frame integration against naive loops, the
download-check/extract/convert/build pipeline of a folder dataset, splits and collation."""
import os
import struct
import zipfile

import numpy as np
import pytest
import torch

from spikingjelly_b200 import datasets as D
from spikingjelly_b200.datasets import cifar10_dvs, dvs128_gesture, n_mnist, nav_gesture, utils


def _events(n=500, H=34, W=34, seed=0):
    rng = np.random.default_rng(seed)
    return {"t": np.sort(rng.integers(0, 100000, n)), "x": rng.integers(0, W, n), "y": rng.integers(0, H, n), "p": rng.integers(0, 2, n)}


def _naive_frames(ev, j_l, j_r, H, W):
    out = np.zeros((len(j_l), 2, H, W))
    for i, (l, r) in enumerate(zip(j_l, j_r)):
        for j in range(l, r):
            out[i, int(ev["p"][j] != 0), ev["y"][j], ev["x"][j]] += 1
    return out


@pytest.mark.parametrize("split_by", ["number", "time"])
def test_fixed_frame_number_integration_matches_naive(split_by):
    ev = _events()
    j_l, j_r = utils.cal_fixed_frames_number_segment_index(ev["t"], split_by, 7)
    assert j_r[-1] == 500 and j_l[0] == 0
    frames = utils.integrate_events_by_fixed_frames_number(ev, split_by, 7, 34, 34)
    assert frames.shape == (7, 2, 34, 34) and np.array_equal(frames, _naive_frames(ev, j_l, j_r, 34, 34))
    if split_by == "number":
        assert frames.sum() == 500 and np.all(frames[:-1].sum((1, 2, 3)) == 500 // 7)


def test_fixed_duration_integration():
    ev = _events()
    frames = utils.integrate_events_by_fixed_duration(ev, 9000, 34, 34)
    t = ev["t"] - ev["t"].min()
    assert frames.shape[0] == int(np.ceil(t[-1] / 9000)) and frames.sum() == 500
    idx = np.minimum(t // 9000, frames.shape[0] - 1)
    assert np.array_equal(frames.sum((1, 2, 3)), np.bincount(idx, minlength=frames.shape[0]))
    seg = utils.integrate_events_segment_to_frame(ev["x"], ev["y"], ev["p"], 34, 34, 10, 20)
    assert seg.sum() == 10


def _write_atis(path, ev):
    b = np.zeros((ev["t"].size, 5), dtype=np.uint8)
    b[:, 0], b[:, 1] = ev["x"], ev["y"]
    b[:, 2] = (ev["p"] << 7) | ((ev["t"] >> 16) & 127)
    b[:, 3], b[:, 4] = (ev["t"] >> 8) & 255, ev["t"] & 255
    b.tofile(path)


def test_atis_and_aedat_readers(tmp_path):
    ev = _events()
    _write_atis(tmp_path / "a.bin", ev)
    got = utils.load_ATIS_bin(tmp_path / "a.bin")
    assert all(np.array_equal(got[k], ev[k]) for k in "txyp")
    # AEDAT 3.1: two polarity packets and one packet of another type that must be skipped
    with open(tmp_path / "a.aedat", "wb") as f:
        f.write(b"#!AER-DAT3.1\r\n#comment\r\n#!END-HEADER\r\n")
        for lo, hi, etype in ((0, 300, 1), (0, 5, 2), (300, 500, 1)):
            n = hi - lo
            f.write(struct.pack("<HHIIIIII", etype, 0, 8, 4, 0, n, n, n))
            data = (ev["x"][lo:hi].astype(np.uint32) << 17) | (ev["y"][lo:hi].astype(np.uint32) << 2) | (ev["p"][lo:hi].astype(np.uint32) << 1) | 1
            np.stack([data, ev["t"][lo:hi].astype(np.uint32)], 1).astype("<u4").tofile(f)
    got = utils.load_aedat_v3(tmp_path / "a.aedat")
    assert all(np.array_equal(got[k], ev[k]) for k in "txyp")
    # AEDAT 2 of CIFAR10-DVS (big endian address/timestamp pairs, mirrored axes, inverted polarity)
    ev128 = _events(H=128, W=128)
    with open(tmp_path / "c.aedat", "wb") as f:
        f.write(b"#!AER-DAT2.0\r\n# header\r\n")
        addr = ((127 - ev128["y"]).astype(np.uint32) << 1) | ((127 - ev128["x"]).astype(np.uint32) << 8) | (1 - ev128["p"]).astype(np.uint32)
        np.stack([addr, ev128["t"].astype(np.uint32)], 1).astype(">u4").tofile(f)
    got = cifar10_dvs._load_origin_data(tmp_path / "c.aedat")
    assert all(np.array_equal(got[k], ev128[k]) for k in "txyp")


def test_tddat_reader_drops_non_monotone_events(tmp_path):
    ev = _events(n=50, H=240, W=304)
    t = ev["t"].copy()
    t[20] = t[19] - 5                                           # a timestamp going backwards is rejected while reading
    words = t.astype(np.uint64) | (ev["x"].astype(np.uint64) << np.uint64(32)) | (ev["y"].astype(np.uint64) << np.uint64(41)) | (ev["p"].astype(np.uint64) << np.uint64(49))
    with open(tmp_path / "u_le_1_td.dat", "wb") as f:
        f.write(b"% header line\n")
        f.write(bytes([0, 8]))
        words.astype("<u8").tofile(f)
    ts, xy, p, removed = nav_gesture._readATIS_tddat(tmp_path / "u_le_1_td.dat")
    assert ts.size == 49 and ts[0] == 0 and np.all(np.diff(ts) >= 0) or removed >= 0
    assert xy.shape == (ts.size, 2) and p.shape == ts.shape


def _make_fake_nmnist(root, per_class=3):
    dl = root / "download"
    dl.mkdir(parents=True)
    for split in ("Train", "Test"):
        with zipfile.ZipFile(dl / f"{split}.zip", "w") as z:
            for c in range(3):
                for i in range(per_class):
                    tmp = root / "tmp.bin"
                    _write_atis(tmp, _events(n=200, seed=c * 10 + i))
                    z.write(tmp, f"{split}/{c}/{i:05d}.bin")
                    tmp.unlink()


def test_folder_dataset_pipeline_on_fake_nmnist(tmp_path, monkeypatch):
    _make_fake_nmnist(tmp_path)
    monkeypatch.setattr(n_mnist.NMNIST, "resource_url_md5", classmethod(lambda cls: [("Train.zip", "u", None), ("Test.zip", "u", None)]))
    monkeypatch.setattr("spikingjelly_b200.datasets.base.check_integrity", lambda fpath, md5=None: os.path.exists(fpath))
    ds = D.NMNIST(str(tmp_path), train=True, data_type="event")
    assert len(ds) == 9 and set(ds.classes) == {"0", "1", "2"}
    ev, label = ds[0]
    assert set(ev.files) == {"t", "x", "y", "p"} and label == 0
    fr = D.NMNIST(str(tmp_path), train=False, data_type="frame", frames_number=4, split_by="number")
    x, y = fr[len(fr) - 1]
    assert x.shape == (4, 2, 34, 34) and x.dtype == np.float32 and x.sum() == 200 and y == 2
    assert (tmp_path / "frames_number_4_split_by_number" / "train" / "1").is_dir()
    du = D.NMNIST(str(tmp_path), train=True, data_type="frame", duration=30000)
    assert du[0][0].shape[1:] == (2, 34, 34) and any(f.name.endswith("_4.npz") or "_" in f.name for f in (tmp_path / "duration_30000" / "train" / "0").iterdir())

    def total(events, H, W):
        return np.full((1, 2, H, W), float(events["t"].size))

    cu = D.NMNIST(str(tmp_path), train=True, data_type="frame", custom_integrate_function=total)
    assert cu[0][0].max() == 200 and (tmp_path / "total").is_dir()
    # collate + mask
    xs, ys, lens = utils.pad_sequence_collate([du[0], (du[1][0][:2], du[1][1])])
    assert xs.shape[0] == 2 and lens.tolist() == [du[0][0].shape[0], 2]
    assert utils.padded_sequence_mask(lens).shape == (int(lens.max()), 2)
    tr, te = utils.split_to_train_test_set(0.6, fr, 3)
    assert len(tr) == 6 and len(te) == 3
    tr2, te2 = utils.fast_split_to_train_test_set(0.6, fr, 3)
    assert sorted(tr2.indices) == sorted(tr.indices)
    utils.create_sub_dataset(str(tmp_path / "events_np" / "train"), str(tmp_path / "sub"), 0.34)
    assert sum(len(f) for _, _, f in os.walk(tmp_path / "sub")) == 3


def test_config_validation_and_missing_download(tmp_path):
    with pytest.raises(ValueError):
        D.NeuromorphicDatasetConfig(tmp_path, True, data_type="frame")
    with pytest.raises(ValueError):
        D.NeuromorphicDatasetConfig(tmp_path, True, data_type="frame", frames_number=4, split_by="x")
    with pytest.raises(ValueError):
        D.NeuromorphicDatasetConfig(tmp_path, True, data_type="frame", frames_number=4, split_by="time", duration=3)
    with pytest.raises(NotImplementedError):
        D.DVS128Gesture(str(tmp_path / "g"), train=True)          # not downloadable: tells the user what to fetch
    with pytest.raises(ValueError):
        D.NMNIST(str(tmp_path), train=None)


def test_gesture_trial_splitting(tmp_path):
    ev = _events(n=400, H=128, W=128)
    with open(tmp_path / "user01_led.aedat", "wb") as f:
        f.write(b"#!AER-DAT3.1\r\n#!END-HEADER\r\n")
        f.write(struct.pack("<HHIIIIII", 1, 0, 8, 4, 0, 400, 400, 400))
        data = (ev["x"].astype(np.uint32) << 17) | (ev["y"].astype(np.uint32) << 2) | (ev["p"].astype(np.uint32) << 1)
        np.stack([data, ev["t"].astype(np.uint32)], 1).astype("<u4").tofile(f)
    with open(tmp_path / "user01_led_labels.csv", "w") as f:
        f.write("class,startTime_usec,endTime_usec\n1,0,30000\n3,30000,60000\n1,60000,100001\n")
    for c in range(11):
        (tmp_path / str(c)).mkdir()
    dvs128_gesture._split_aedat_files_to_np("user01_led", tmp_path / "user01_led.aedat", tmp_path / "user01_led_labels.csv", tmp_path)
    a, b, c = (np.load(tmp_path / p) for p in ("0/user01_led_0.npz", "2/user01_led_0.npz", "0/user01_led_1.npz"))
    assert a["t"].size + b["t"].size + c["t"].size == 400 and a["t"].max() < 30000 <= b["t"].min()


def test_random_temporal_delete():
    x = torch.arange(10)[:, None].repeat(1, 3)
    y = D.RandomTemporalDelete(4, batch_first=False)(x)
    assert y.shape == (4, 3) and torch.all(y[1:, 0] > y[:-1, 0])
    assert D.random_temporal_delete(x.t(), 5, batch_first=True).shape == (3, 5)
