"""Seekable read-only file object over an HTTP server that honours ``Range`` requests.

Used to pull single members out of large remote archives (zip central directory, then the
member's bytes) without downloading the archive.  Behaviour follows the reference's reader
(``prism_infer/analysis/http_range_reader.py:22-236``): a strict ``Content-Range`` parser, a
one-byte probe at construction that also checks the recorded object size, fixed-size chunks
kept in a small LRU, every chunk fetched through the original URL (signed redirects are
valid for one byte interval only), retry with exponential back-off on transport errors and
on 429/5xx, and counters for requests, bytes and cache hits.  This version uses
``urllib.request`` so it has no third-party dependency.
"""

from __future__ import annotations

import io
import re
import time
import urllib.error
import urllib.request
from collections import OrderedDict

DEFAULT_RANGE_CHUNK_BYTES = 8 * 1024 * 1024
DEFAULT_CACHE_CHUNKS = 4
RETRY_STATUS = (429, 500, 502, 503, 504)
_CONTENT_RANGE = re.compile(r"bytes (\d+)-(\d+)/(\d+)")


def parse_content_range(value: str | None) -> tuple[int, int, int]:
    """``bytes start-end/total`` -> ``(start, end, total)``; anything else raises."""
    if value is None:
        raise ValueError("partial-content response carries no Content-Range header")
    m = _CONTENT_RANGE.fullmatch(value.strip())
    if m is None:
        raise ValueError(f"malformed Content-Range header: {value!r}")
    start, end, total = (int(g) for g in m.groups())
    if end < start or end >= total:
        raise ValueError(f"inconsistent Content-Range header: {value!r}")
    return start, end, total


def _positive_int(name: str, value: object) -> int:
    if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
        raise ValueError(f"{name} must be a positive integer")
    return value


class HTTPRangeReader(io.RawIOBase):
    def __init__(self, url: str, *, expected_size: int, chunk_bytes: int = DEFAULT_RANGE_CHUNK_BYTES,
                 cache_chunks: int = DEFAULT_CACHE_CHUNKS, timeout_seconds: float = 60.0, retries: int = 5,
                 backoff_seconds: float = 0.5) -> None:
        super().__init__()
        if not url:
            raise ValueError("url must be non-empty")
        self._url = url
        self._size = _positive_int("expected_size", expected_size)
        self._chunk = _positive_int("chunk_bytes", chunk_bytes)
        self._cap = _positive_int("cache_chunks", cache_chunks)
        self._retries = _positive_int("retries", retries)
        self._timeout = float(timeout_seconds)
        self._backoff = float(backoff_seconds)
        self._pos = 0
        self._cache: OrderedDict[int, bytes] = OrderedDict()
        self._resolved = url
        self.range_requests = 0
        self.range_response_bytes = 0
        self.cache_hits = 0
        if len(self._get(0, 0)) != 1:  # probe: range support and recorded size
            raise OSError("one-byte range probe returned a payload of the wrong length")

    # ------------------------------------------------------------------ transport
    @property
    def size(self) -> int:
        return self._size

    @property
    def resolved_url(self) -> str:
        return self._resolved

    def _get(self, start: int, end: int) -> bytes:
        req = urllib.request.Request(self._url, headers={"Range": f"bytes={start}-{end}", "Accept-Encoding": "identity"})
        last: BaseException | None = None
        for attempt in range(self._retries + 1):
            try:
                with urllib.request.urlopen(req, timeout=self._timeout) as resp:
                    status, header, final = resp.status, resp.headers.get("Content-Range"), resp.geturl()
                    body = resp.read()
            except urllib.error.HTTPError as exc:
                if exc.code in RETRY_STATUS and attempt < self._retries:
                    last = exc
                    time.sleep(min(self._backoff * (2 ** attempt), 8.0))
                    continue
                raise OSError(f"range request {start}-{end} failed with HTTP {exc.code}") from exc
            except (urllib.error.URLError, TimeoutError, ConnectionError) as exc:
                if attempt < self._retries:
                    last = exc
                    time.sleep(min(self._backoff * (2 ** attempt), 8.0))
                    continue
                raise
            if status != 206:
                raise OSError(f"server ignored the Range header: status={status}, requested={start}-{end}")
            got_start, got_end, total = parse_content_range(header)
            if (got_start, got_end) != (start, end):
                raise OSError(f"server answered bytes {got_start}-{got_end}, requested {start}-{end}")
            if total != self._size:
                raise OSError(f"remote object has {total} bytes, recorded size is {self._size}")
            if len(body) != end - start + 1:
                raise OSError(f"range payload has {len(body)} bytes, expected {end - start + 1}")
            self._resolved = final
            return body
        raise OSError(f"range request {start}-{end} gave up after {self._retries} retries: {last}")

    def _chunk_bytes(self, index: int) -> bytes:
        hit = self._cache.get(index)
        if hit is not None:
            self._cache.move_to_end(index)
            self.cache_hits += 1
            return hit
        start = index * self._chunk
        if start >= self._size:
            return b""
        data = self._get(start, min(start + self._chunk, self._size) - 1)
        self.range_requests += 1
        self.range_response_bytes += len(data)
        self._cache[index] = data
        while len(self._cache) > self._cap:
            self._cache.popitem(last=False)
        return data

    # ------------------------------------------------------------------ io.RawIOBase
    def readable(self) -> bool:
        return True

    def seekable(self) -> bool:
        return True

    def tell(self) -> int:
        return self._pos

    def seek(self, offset: int, whence: int = io.SEEK_SET) -> int:
        base = {io.SEEK_SET: 0, io.SEEK_CUR: self._pos, io.SEEK_END: self._size}.get(whence)
        if base is None:
            raise ValueError(f"unsupported whence: {whence}")
        target = base + offset
        if target < 0:
            raise ValueError("negative seek position")
        self._pos = target
        return target

    def read(self, size: int = -1) -> bytes:
        if self.closed:
            raise ValueError("read from a closed reader")
        end = self._size if size is None or size < 0 else min(self._size, self._pos + size)
        parts = []
        while self._pos < end:
            index, inner = divmod(self._pos, self._chunk)
            piece = self._chunk_bytes(index)[inner:inner + (end - self._pos)]
            if not piece:
                break
            parts.append(piece)
            self._pos += len(piece)
        return b"".join(parts)

    def readinto(self, buffer) -> int:
        data = self.read(len(buffer))
        buffer[:len(data)] = data
        return len(data)

    def close(self) -> None:
        self._cache.clear()
        super().close()
