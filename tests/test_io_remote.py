"""Remote IO paths against in-memory fakes of the object-store SDKs (no network): S3-compatible, GCS, HTTP, and a
user-registered scheme; plus reading a numpy token file and a checkpoint through a URL."""

import sys
import types

import numpy as np
import pytest
import torch

from olmo_core_b200 import io


class _FakeS3:
    """The handful of boto3 client calls the S3 client uses, over a dict {(bucket, key): bytes}."""

    def __init__(self, store):
        self.store = store

    def head_object(self, Bucket, Key):
        if (Bucket, Key) not in self.store:
            raise RuntimeError("An error occurred (404) when calling the HeadObject operation: Not Found")
        return {"ContentLength": len(self.store[(Bucket, Key)])}

    def get_object(self, Bucket, Key, Range):
        if (Bucket, Key) not in self.store:
            raise RuntimeError("NoSuchKey")
        lo, hi = (int(v) for v in Range.split("=")[1].split("-"))
        data = self.store[(Bucket, Key)][lo:hi + 1]
        return {"Body": types.SimpleNamespace(read=lambda: data)}

    def upload_file(self, filename, Bucket, Key):
        self.store[(Bucket, Key)] = open(filename, "rb").read()

    def delete_object(self, Bucket, Key):
        self.store.pop((Bucket, Key), None)

    def get_paginator(self, name):
        assert name == "list_objects_v2"
        store = self.store

        class P:
            def paginate(self, Bucket, Prefix, Delimiter=None):
                keys = sorted(k for (b, k) in store if b == Bucket and k.startswith(Prefix))
                if Delimiter is None:
                    yield {"Contents": [{"Key": k} for k in keys]}
                    return
                files, dirs = [], set()
                for k in keys:
                    rest = k[len(Prefix):]
                    if Delimiter in rest:
                        dirs.add(Prefix + rest.split(Delimiter)[0] + Delimiter)
                    else:
                        files.append(k)
                yield {"Contents": [{"Key": k} for k in files], "CommonPrefixes": [{"Prefix": d} for d in sorted(dirs)]}

        return P()


@pytest.fixture
def fake_s3(monkeypatch):
    store = {}
    boto3 = types.ModuleType("boto3")
    boto3.Session = lambda profile_name=None: types.SimpleNamespace(client=lambda *a, **k: _FakeS3(store))
    botocore = types.ModuleType("botocore")
    botocore_config = types.ModuleType("botocore.config")
    botocore_config.Config = lambda **k: None
    monkeypatch.setitem(sys.modules, "boto3", boto3)
    monkeypatch.setitem(sys.modules, "botocore", botocore)
    monkeypatch.setitem(sys.modules, "botocore.config", botocore_config)
    for scheme in ("s3", "r2", "weka"):
        io._CLIENTS.pop(scheme, None)
    yield store
    for scheme in ("s3", "r2", "weka"):
        io._CLIENTS.pop(scheme, None)


@pytest.mark.parametrize("scheme", ["s3", "r2", "weka"])
def test_s3_compatible_round_trip(fake_s3, tmp_path, scheme):
    url = f"{scheme}://bucket/run/step10/model.bin"
    assert not io.file_exists(url)
    io.write_bytes(url, b"0123456789")
    assert io.file_exists(url) and io.get_file_size(url) == 10
    assert io.get_bytes_range(url, 3, 4) == b"3456"
    assert io.read_text(url) == "0123456789"
    with pytest.raises(FileExistsError):
        io.write_bytes(url, b"x", overwrite=False)
    io.write_text(f"{scheme}://bucket/run/step10/sub/meta.json", "{}")
    io.write_text(f"{scheme}://bucket/run/config.json", "{}")
    flat = sorted(io.list_directory(f"{scheme}://bucket/run"))
    assert flat == [f"{scheme}://bucket/run/config.json", f"{scheme}://bucket/run/step10"]
    deep = sorted(io.list_directory(f"{scheme}://bucket/run", recurse=True))
    assert deep == [f"{scheme}://bucket/run/config.json", url, f"{scheme}://bucket/run/step10/sub/meta.json"]
    assert sorted(io.glob_directory(f"{scheme}://bucket/run/*/*.bin")) == [url]
    assert not io.dir_is_empty(f"{scheme}://bucket/run") and io.dir_is_empty(f"{scheme}://bucket/other")
    # store -> local, local -> store, store -> store
    local = tmp_path / "copy.bin"
    io.copy_file(url, local)
    assert local.read_bytes() == b"0123456789"
    io.copy_file(local, f"{scheme}://bucket/copy.bin")
    io.copy_file(f"{scheme}://bucket/copy.bin", f"{scheme}://bucket/copy2.bin")
    assert fake_s3[("bucket", "copy2.bin")] == b"0123456789"
    io.copy_dir(f"{scheme}://bucket/run", tmp_path / "mirror")
    assert (tmp_path / "mirror" / "step10" / "sub" / "meta.json").read_text() == "{}"
    io.remove_file(url)
    assert not io.file_exists(url)
    with pytest.raises(FileNotFoundError):
        io.get_file_size(url)
    io.clear_directory(f"{scheme}://bucket/run")
    assert io.dir_is_empty(f"{scheme}://bucket/run")


def test_gcs_client_against_fake_sdk(monkeypatch, tmp_path):
    blobs = {}

    class Blob:
        def __init__(self, bucket, name):
            self.key, self.name = (bucket, name), name

        def exists(self):
            return self.key in blobs

        def reload(self):
            self.size = len(blobs[self.key])

        def download_as_bytes(self, start, end):
            return blobs[self.key][start:end + 1]

        def upload_from_filename(self, filename):
            blobs[self.key] = open(filename, "rb").read()

        def delete(self):
            blobs.pop(self.key, None)

    class Listing(list):
        prefixes = ()

    class Client:
        def bucket(self, name):
            return types.SimpleNamespace(blob=lambda key: Blob(name, key))

        def list_blobs(self, bucket, prefix, delimiter):
            names = sorted(k for (b, k) in blobs if b == bucket and k.startswith(prefix))
            out = Listing(Blob(bucket, n) for n in names if delimiter is None or delimiter not in n[len(prefix):])
            out.prefixes = sorted({prefix + n[len(prefix):].split("/")[0] + "/" for n in names
                                   if delimiter is not None and delimiter in n[len(prefix):]})
            return out

    google = types.ModuleType("google")
    cloud = types.ModuleType("google.cloud")
    storage = types.ModuleType("google.cloud.storage")
    storage.Client = Client
    cloud.storage = storage
    google.cloud = cloud
    for name, mod in (("google", google), ("google.cloud", cloud), ("google.cloud.storage", storage)):
        monkeypatch.setitem(sys.modules, name, mod)
    io._CLIENTS.pop("gs", None)
    try:
        io.write_bytes("gs://b/a/x.npy", b"abcdef")
        io.write_bytes("gs://b/a/deep/y.npy", b"zz")
        assert io.get_file_size("gs://b/a/x.npy") == 6 and io.get_bytes_range("gs://b/a/x.npy", 1, 3) == b"bcd"
        assert sorted(io.list_directory("gs://b/a")) == ["gs://b/a/deep", "gs://b/a/x.npy"]
        assert sorted(io.list_directory("gs://b/a", recurse=True)) == ["gs://b/a/deep/y.npy", "gs://b/a/x.npy"]
        with pytest.raises(FileExistsError):
            io.write_bytes("gs://b/a/x.npy", b"q", overwrite=False)
        io.remove_file("gs://b/a/x.npy")
        assert not io.file_exists("gs://b/a/x.npy")
    finally:
        io._CLIENTS.pop("gs", None)


def test_http_range_reads(monkeypatch):
    from olmo_core_b200.exceptions import OLMoInvalidRangeRequestError, OLMoNetworkError

    payload = bytes(range(200))

    def head(url, **kw):
        ok = url.endswith("/file")
        return types.SimpleNamespace(status_code=200 if ok else 404, headers={"content-length": str(len(payload))})

    def get(url, headers, **kw):
        if url.endswith("/broken"):
            return types.SimpleNamespace(status_code=503, content=b"")
        if not url.endswith(("/file", "/norange")):
            return types.SimpleNamespace(status_code=404, content=b"")
        lo, hi = (int(v) for v in headers["Range"].split("=")[1].split("-"))
        if lo >= len(payload):
            return types.SimpleNamespace(status_code=416, content=b"")
        if url.endswith("/norange"):  # a server that ignores Range and sends everything
            return types.SimpleNamespace(status_code=200, content=payload)
        return types.SimpleNamespace(status_code=206, content=payload[lo:hi + 1])

    requests = types.ModuleType("requests")
    requests.head, requests.get = head, get
    monkeypatch.setitem(sys.modules, "requests", requests)
    assert io.file_exists("https://host/file") and not io.file_exists("https://host/missing")
    assert io.get_file_size("https://host/file") == 200
    assert io.get_bytes_range("https://host/file", 10, 5) == payload[10:15]
    assert io.get_bytes_range("https://host/norange", 10, 5) == payload[10:15]
    with pytest.raises(FileNotFoundError):
        io.get_bytes_range("https://host/missing", 0, 1)
    with pytest.raises(OLMoInvalidRangeRequestError):
        io.get_bytes_range("https://host/file", 500, 5)
    with pytest.raises(OLMoNetworkError):
        io.get_bytes_range.__wrapped__("https://host/broken", 0, 5) if hasattr(io.get_bytes_range, "__wrapped__") \
            else io.get_bytes_range("https://host/broken", 0, 5)


class _MemClient(io.SchemeClient):
    scheme = "mem"

    def __init__(self):
        self.files = {}

    def exists(self, url):
        return url in self.files

    def size(self, url):
        if url not in self.files:
            raise FileNotFoundError(url)
        return len(self.files[url])

    def read_range(self, url, start, length):
        return self.files[url][start:start + length]

    def upload(self, source, url, overwrite):
        if not overwrite and url in self.files:
            raise FileExistsError(url)
        self.files[url] = source.read_bytes()

    def delete(self, url):
        self.files.pop(url, None)

    def list(self, url, recurse):
        prefix = url.rstrip("/") + "/"
        out = set()
        for f in self.files:
            if f.startswith(prefix):
                rest = f[len(prefix):]
                out.add(f if (recurse or "/" not in rest) else prefix + rest.split("/")[0])
        return sorted(out)


@pytest.fixture
def mem_store():
    client = _MemClient()
    io.register_scheme_client("mem", lambda: client)
    yield client
    io._CLIENT_FACTORIES.pop("mem", None)
    io._CLIENTS.pop("mem", None)


def test_numpy_dataset_reads_token_files_through_a_url(mem_store, tmp_path):
    from olmo_core_b200.data import NumpyFSLDatasetConfig, TokenizerConfig

    tokens = np.arange(1, 1001, dtype=np.uint16)
    tokens[99::100] = 0  # an end-of-sequence token every 100 tokens
    local = tmp_path / "part-0.npy"
    tokens.tofile(local)
    io.upload(local, "mem://data/part-0.npy")
    tok = TokenizerConfig(vocab_size=2048, eos_token_id=0, pad_token_id=0)
    ds = NumpyFSLDatasetConfig(paths=["mem://data/part-0.npy"], sequence_length=64, tokenizer=tok,
                               work_dir=str(tmp_path / "work")).build()
    ds.prepare() if hasattr(ds, "prepare") else None
    assert len(ds) == 1000 // 64
    np.testing.assert_array_equal(np.asarray(ds[1]["input_ids"]), tokens[64:128].astype(np.int64))


def test_checkpoint_saves_to_and_loads_from_a_url(mem_store, tmp_path):
    from olmo_core_b200.distributed.checkpoint import load_model_and_optim_state, save_model_and_optim_state

    torch.manual_seed(0)
    model = torch.nn.Linear(8, 4)
    save_model_and_optim_state("mem://ckpt/step1", model)
    assert any(f.endswith(".metadata") or ".metadata" in f for f in mem_store.files)
    other = torch.nn.Linear(8, 4)
    load_model_and_optim_state("mem://ckpt/step1", other)
    assert torch.equal(other.weight, model.weight) and torch.equal(other.bias, model.bias)
