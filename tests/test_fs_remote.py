"""The remote back-ends of ``olmax_b200.fs`` (S3 / R2 / Weka, GCS, HTTP) against in-memory fakes of their SDKs: size,
range reads, upload with and without overwrite, existence, removal, listing (flat and recursive, paginated), the
shallow-prefix guard of ``clear_directory`` and the back-off of ``retriable``.  Mirrors what the reference checks against
real buckets in ``src/test/fs_test.py:41-105``."""

import sys
import types

import pytest

from olmax_b200 import fs
from olmax_b200.exceptions import OLMaxEnvironmentError, OLMaxNetworkError, OLMaxUploadError


# ----------------------------------------------------------------------------------------------------------------------
# fakes
# ----------------------------------------------------------------------------------------------------------------------
class FakeS3Client:
    """The five boto3 client calls the back-end uses, over a dict {(bucket, key): bytes}; listings come in pages of 2."""

    def __init__(self, store, calls):
        self.store, self.calls = store, calls

    def head_object(self, Bucket, Key):
        self.calls.append(("head", Bucket, Key))
        if (Bucket, Key) not in self.store:
            raise KeyError("404")
        return {"ContentLength": len(self.store[(Bucket, Key)])}

    def get_object(self, Bucket, Key, Range):
        lo, hi = (int(x) for x in Range[len("bytes="):].split("-"))
        data = self.store[(Bucket, Key)][lo : hi + 1]
        return {"Body": types.SimpleNamespace(read=lambda: data)}

    def upload_file(self, filename, Bucket, Key):
        with open(filename, "rb") as f:
            self.store[(Bucket, Key)] = f.read()

    def delete_object(self, Bucket, Key):
        self.store.pop((Bucket, Key), None)

    def list_objects_v2(self, Bucket, Prefix, Delimiter=None, ContinuationToken=None):
        keys = sorted(k for (b, k) in self.store if b == Bucket and k.startswith(Prefix))
        contents, prefixes = [], []
        for k in keys:
            rest = k[len(Prefix):]
            if Delimiter and Delimiter in rest:
                p = Prefix + rest.split(Delimiter)[0] + Delimiter
                if p not in prefixes:
                    prefixes.append(p)
            else:
                contents.append(k)
        start = int(ContinuationToken or 0)
        page = contents[start : start + 2]
        more = start + 2 < len(contents)
        out = {"Contents": [{"Key": k} for k in page], "IsTruncated": more}
        if more:
            out["NextContinuationToken"] = str(start + 2)
        else:
            out["CommonPrefixes"] = [{"Prefix": p} for p in prefixes]
        return out


@pytest.fixture
def s3(monkeypatch):
    store, calls, sessions = {}, [], []

    class Session:
        def __init__(self, profile_name=None):
            sessions.append(profile_name)

        def client(self, name, config=None, **kw):
            sessions.append(kw)
            return FakeS3Client(store, calls)

    monkeypatch.setitem(sys.modules, "boto3", types.SimpleNamespace(Session=Session))
    monkeypatch.setitem(sys.modules, "botocore", types.ModuleType("botocore"))
    monkeypatch.setitem(sys.modules, "botocore.config", types.SimpleNamespace(Config=lambda **kw: kw))
    monkeypatch.setattr(fs, "_BACKENDS", {})
    return types.SimpleNamespace(store=store, calls=calls, sessions=sessions)


class FakeBlob:
    def __init__(self, store, bucket, name):
        self.store, self.bucket, self.name, self.size = store, bucket, name, None

    def reload(self):
        self.size = len(self.store[(self.bucket, self.name)])

    def download_as_bytes(self, start, end):
        return self.store[(self.bucket, self.name)][start : end + 1]

    def exists(self):
        return (self.bucket, self.name) in self.store

    def upload_from_filename(self, filename):
        with open(filename, "rb") as f:
            self.store[(self.bucket, self.name)] = f.read()

    def delete(self):
        del self.store[(self.bucket, self.name)]


@pytest.fixture
def gcs(monkeypatch):
    store = {}

    class Listing(list):
        prefixes = ()

    class Client:
        def bucket(self, name):
            return types.SimpleNamespace(blob=lambda key: FakeBlob(store, name, key))

        def list_blobs(self, bucket, prefix, delimiter):
            out, prefixes = Listing(), []
            for (b, k) in sorted(store):
                if b != bucket or not k.startswith(prefix):
                    continue
                rest = k[len(prefix):]
                if delimiter and delimiter in rest:
                    p = prefix + rest.split(delimiter)[0] + delimiter
                    if p not in prefixes:
                        prefixes.append(p)
                else:
                    out.append(types.SimpleNamespace(name=k))
            out.prefixes = prefixes
            return out

    google = types.ModuleType("google")
    cloud = types.ModuleType("google.cloud")
    storage = types.SimpleNamespace(Client=Client)
    cloud.storage = storage
    google.cloud = cloud
    monkeypatch.setitem(sys.modules, "google", google)
    monkeypatch.setitem(sys.modules, "google.cloud", cloud)
    monkeypatch.setitem(sys.modules, "google.cloud.storage", storage)
    monkeypatch.setattr(fs, "_BACKENDS", {})
    return store


# ----------------------------------------------------------------------------------------------------------------------
# S3-compatible stores
# ----------------------------------------------------------------------------------------------------------------------
def test_s3_round_trip_listing_and_clear(s3, tmp_path):
    src = tmp_path / "a.bin"
    src.write_bytes(bytes(range(200)))
    fs.upload(src, "s3://bkt/run/step1/a.bin")
    assert fs.file_exists("s3://bkt/run/step1/a.bin") and not fs.file_exists("s3://bkt/run/step1/missing")
    assert fs.get_file_size("s3://bkt/run/step1/a.bin") == 200
    assert fs.get_bytes_range("s3://bkt/run/step1/a.bin", 10, 5) == bytes(range(10, 15))
    with pytest.raises(FileExistsError):
        fs.upload(src, "s3://bkt/run/step1/a.bin")
    src.write_bytes(b"new")
    fs.upload(src, "s3://bkt/run/step1/a.bin", save_overwrite=True)
    assert fs.read_text("s3://bkt/run/step1/a.bin") == "new"
    for name in ("b", "c", "d"):
        fs.write_text(f"s3://bkt/run/step1/{name}.txt", name)
    fs.write_text("s3://bkt/run/step1/sub/e.txt", "e")
    fs.write_text("s3://bkt/run/step2/f.txt", "f")
    # flat listing: files of the prefix (over several pages) plus its sub-"directories"
    assert fs.list_directory("s3://bkt/run/step1") == sorted(
        [f"s3://bkt/run/step1/{n}" for n in ("a.bin", "b.txt", "c.txt", "d.txt", "sub")])
    assert "s3://bkt/run/step1/sub/e.txt" in fs.list_directory("s3://bkt/run/step1", recurse=True)
    assert fs.glob_directory("s3://bkt/run/step*/*.txt") == sorted(
        ["s3://bkt/run/step1/b.txt", "s3://bkt/run/step1/c.txt", "s3://bkt/run/step1/d.txt", "s3://bkt/run/step2/f.txt"])
    assert not fs.dir_is_empty("s3://bkt/run/step1") and fs.dir_is_empty("s3://bkt/run/nothing")
    # local directory -> remote prefix, remote file -> local file
    (tmp_path / "d" / "x").mkdir(parents=True)
    (tmp_path / "d" / "x" / "y.txt").write_text("y")
    fs.copy_dir(tmp_path / "d", "s3://bkt/run/copied")
    assert fs.read_text("s3://bkt/run/copied/x/y.txt") == "y"
    fs.copy_file("s3://bkt/run/copied/x/y.txt", tmp_path / "back.txt")
    assert (tmp_path / "back.txt").read_text() == "y"
    fs.remove_file("s3://bkt/run/step2/f.txt")
    assert not fs.file_exists("s3://bkt/run/step2/f.txt")
    # a shallow prefix is refused unless forced; a deep one is emptied
    with pytest.raises(ValueError, match="shallow"):
        fs.clear_directory("s3://bkt/run")
    fs.clear_directory("s3://bkt/run/step1")
    assert fs.dir_is_empty("s3://bkt/run/step1") and fs.file_exists("s3://bkt/run/copied/x/y.txt")
    fs.clear_directory("s3://bkt/run", force=True)
    assert not s3.store


def test_r2_and_weka_need_and_use_their_endpoint(s3, monkeypatch, tmp_path):
    monkeypatch.delenv("R2_ENDPOINT_URL", raising=False)
    with pytest.raises(OLMaxEnvironmentError, match="R2_ENDPOINT_URL"):
        fs.file_exists("r2://bkt/a/b")
    monkeypatch.setenv("WEKA_ENDPOINT_URL", "https://weka.example:9000")
    monkeypatch.setenv("WEKA_PROFILE", "weka-profile")
    fs.init_client("weka://bkt/a/b")
    assert "weka-profile" in s3.sessions and {"endpoint_url": "https://weka.example:9000"} in s3.sessions
    fs.write_text("weka://bkt/a/b.txt", "w")
    assert fs.list_directory("weka://bkt/a") == ["weka://bkt/a/b.txt"]


def test_missing_sdk_is_reported(monkeypatch):
    monkeypatch.setitem(sys.modules, "boto3", None)   # import boto3 -> ImportError
    monkeypatch.setattr(fs, "_BACKENDS", {})
    with pytest.raises(OLMaxEnvironmentError, match="boto3"):
        fs.get_file_size("s3://bkt/a/b")
    with pytest.raises(NotImplementedError):
        fs.get_file_size("ftp://host/a")


# ----------------------------------------------------------------------------------------------------------------------
# GCS
# ----------------------------------------------------------------------------------------------------------------------
def test_gcs_round_trip(gcs, tmp_path):
    src = tmp_path / "a.bin"
    src.write_bytes(b"0123456789")
    fs.copy_file(src, "gs://bkt/ckpt/step3/a.bin")
    assert fs.get_file_size("gs://bkt/ckpt/step3/a.bin") == 10
    assert fs.get_bytes_range("gs://bkt/ckpt/step3/a.bin", 2, 3) == b"234"
    with pytest.raises(FileExistsError):
        fs.copy_file(src, "gs://bkt/ckpt/step3/a.bin")
    fs.copy_file(src, "gs://bkt/ckpt/step3/a.bin", save_overwrite=True)
    fs.write_text("gs://bkt/ckpt/step3/items/meta.json", "{}")
    assert fs.list_directory("gs://bkt/ckpt/step3") == ["gs://bkt/ckpt/step3/a.bin", "gs://bkt/ckpt/step3/items"]
    assert fs.list_directory("gs://bkt/ckpt/step3", recurse=True) == [
        "gs://bkt/ckpt/step3/a.bin", "gs://bkt/ckpt/step3/items/meta.json"]
    assert fs.join_path("gs://bkt/ckpt/", "step3", "a.bin") == "gs://bkt/ckpt/step3/a.bin"
    fs.clear_directory("gs://bkt/ckpt/step3")
    assert not gcs


# ----------------------------------------------------------------------------------------------------------------------
# HTTP
# ----------------------------------------------------------------------------------------------------------------------
def test_http_reads_and_refuses_writes(monkeypatch, tmp_path):
    body = bytes(range(100))
    seen = []

    def head(url, allow_redirects=True):
        seen.append(("HEAD", url))
        ok = url.endswith("/data/file.npy")
        return types.SimpleNamespace(status_code=200 if ok else 404, headers={"Content-Length": str(len(body))})

    def get(url, headers):
        lo, hi = (int(x) for x in headers["Range"][len("bytes="):].split("-"))
        code = 206 if url.endswith("/data/file.npy") else (503 if "flaky" in url else 404)
        return types.SimpleNamespace(status_code=code, content=body[lo : hi + 1])

    monkeypatch.setattr(fs, "_BACKENDS", {})
    be = fs._backend("https")
    monkeypatch.setattr(be, "requests", types.SimpleNamespace(head=head, get=get))
    monkeypatch.setitem(fs._BACKENDS, "http", be)
    assert fs.get_file_size("https://host.example/data/file.npy") == 100
    assert fs.get_bytes_range("http://host.example/data/file.npy", 90, 10) == body[90:]
    assert ("HEAD", "https://host.example/data/file.npy") in seen
    assert fs.file_exists("https://host.example/data/file.npy") and not fs.file_exists("https://host.example/nope")
    with pytest.raises(FileNotFoundError):
        fs.get_bytes_range("https://host.example/nope", 0, 1)
    monkeypatch.setattr(fs.time, "sleep", lambda s: None)
    with pytest.raises(OLMaxNetworkError, match="503"):
        fs.get_bytes_range("https://host.example/flaky", 0, 1)
    (tmp_path / "f").write_text("x")
    with pytest.raises(OLMaxUploadError):
        fs.upload(tmp_path / "f", "https://host.example/data/f")


# ----------------------------------------------------------------------------------------------------------------------
# retriable
# ----------------------------------------------------------------------------------------------------------------------
def test_retriable_backs_off_exponentially_and_gives_up(monkeypatch):
    sleeps = []
    monkeypatch.setattr(fs.time, "sleep", sleeps.append)
    attempts = {"n": 0}

    @fs.retriable(max_attempts=4, max_backoff=1.5)
    def flaky(fail_times):
        attempts["n"] += 1
        if attempts["n"] <= fail_times:
            raise OLMaxNetworkError("try again")
        return attempts["n"]

    assert flaky(2) == 3 and sleeps == [0.5, 1.0]
    attempts["n"], sleeps[:] = 0, []
    with pytest.raises(OLMaxNetworkError):
        flaky(10)
    assert attempts["n"] == 4 and sleeps == [0.5, 1.0, 1.5]   # capped by max_backoff

    @fs.retriable(retry_condition=lambda e: "transient" in str(e))
    def picky():
        attempts["n"] += 1
        raise OSError("permanent")

    attempts["n"] = 0
    with pytest.raises(OSError):
        picky()
    assert attempts["n"] == 1   # not retried: the condition said no

    @fs.retriable()
    def missing():
        attempts["n"] += 1
        raise FileNotFoundError("x")

    attempts["n"] = 0
    with pytest.raises(FileNotFoundError):
        missing()
    assert attempts["n"] == 1   # a missing file is an answer, not a failure
