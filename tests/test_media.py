"""Media resolver policy: inline data, allow-listed files and hosts, size and type checks, caching."""
import base64
import os

import pytest

from cubic_serve_b200.inputs.media import MediaError, MediaPolicy, MediaResolver, sniff

PNG = b"\x89PNG\r\n\x1a\n" + b"\x00" * 32
JPEG = b"\xff\xd8\xff\xe0" + b"\x00" * 32
MP4 = b"\x00\x00\x00\x18ftypmp42" + b"\x00" * 32


def _data(mime, raw):
    return f"data:{mime};base64,{base64.b64encode(raw).decode()}"


def test_inline_data_is_decoded_typed_and_cached():
    r = MediaResolver()
    m = r.resolve(_data("image/png", PNG))
    assert (m.kind, m.mime, m.source, len(m.sha256)) == ("image", "image/png", "data", 64) and m.data == PNG
    assert r.resolve(_data("image/png", PNG)) is m and r.stats == {"resolved": 1, "cache_hits": 1}
    assert r.resolve(_data("video/mp4", MP4), "video").mime == "video/mp4"
    assert sniff(b"RIFF\x00\x00\x00\x00WEBPVP8 ") == "image/webp" and sniff(b"hello") is None
    for bad in ("data:image/png;base64", "data:image/png," + "AAAA", _data("image/png", PNG)[:-3] + "!!!",
                _data("image/jpeg", PNG), _data("image/png", b"not an image"), _data("image/png", MP4), "ftp://x/y.png", ""):
        with pytest.raises(MediaError):
            r.resolve(bad)
    with pytest.raises(MediaError, match="larger"):
        MediaResolver(MediaPolicy(max_bytes=16)).resolve(_data("image/png", PNG))
    small = MediaResolver(MediaPolicy(cache_entries=1))
    small.resolve(_data("image/png", PNG))
    small.resolve(_data("image/jpeg", JPEG))
    assert len(small._cache) == 1


def test_files_only_below_allowed_roots(tmp_path):
    root, outside = tmp_path / "media", tmp_path / "secret"
    root.mkdir()
    outside.mkdir()
    (root / "a.png").write_bytes(PNG)
    (outside / "b.png").write_bytes(PNG)
    os.symlink(outside / "b.png", root / "link.png")
    with pytest.raises(MediaError, match="not enabled"):
        MediaResolver().resolve(str(root / "a.png"))
    r = MediaResolver(MediaPolicy(file_roots=(str(root),)))
    assert r.resolve(f"file://{root}/a.png").source == "file" and r.resolve(str(root / "a.png")).mime == "image/png"
    for bad in (str(outside / "b.png"), f"file://{root}/../secret/b.png", str(root / "link.png"), str(root / "missing.png")):
        with pytest.raises(MediaError):
            r.resolve(bad)


def test_remote_media_only_from_allowed_hosts():
    calls = []

    def fetch(url, timeout, max_bytes):
        calls.append((url, timeout, max_bytes))
        return "image/jpeg; charset=binary", JPEG

    r = MediaResolver(MediaPolicy(http_hosts=("cdn.example.com",), timeout_seconds=3.0), fetch=fetch)
    m = r.resolve("https://cdn.example.com/x.jpg")
    assert m.source == "http" and m.mime == "image/jpeg" and calls == [("https://cdn.example.com/x.jpg", 3.0, 32 << 20)]
    with pytest.raises(MediaError, match="not enabled"):
        r.resolve("https://evil.example.org/x.jpg")
    with pytest.raises(MediaError, match="not enabled"):
        MediaResolver(fetch=fetch).resolve("http://cdn.example.com/x.jpg")
    lying = MediaResolver(MediaPolicy(http_hosts=("h",)), fetch=lambda u, t, m: ("image/png", JPEG))
    with pytest.raises(MediaError, match="does not match"):
        lying.resolve("http://h/x")
