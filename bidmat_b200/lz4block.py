"""The stream format of BIDMat's `.lz4` matrix files.

BIDMat writes them with lz4-java's LZ4BlockOutputStream and reads them with
LZ4BlockInputStream (src/main/scala/BIDMat/HMat.scala:86-107; dependency
net.jpountz.lz4:lz4:1.3, pom.xml:151-154, not vendored in the BIDMat tree).
That library's stream is NOT the LZ4 frame format of the `lz4` command line
tool.  Restated here from its published description:

  stream  = block* end-block
  block   = "LZ4Block" (8 bytes)
            token (1 byte)      high nibble: 0x10 raw, 0x20 LZ4-compressed;
                                low nibble: level, block size = 1 << (10 + level)
            compressed length   int32 little-endian
            original length     int32 little-endian
            checksum            int32 little-endian: XXH32 of the original bytes,
                                seed 0x9747b28c, of which lz4-java 1.3 keeps the
                                low 28 bits
            payload             `compressed length` bytes
  end-block = a block with both lengths 0 (checksum 0, no payload)

The payload of a compressed block is one LZ4 block (the public block format:
sequences of token, literal run, 2-byte little-endian match offset, match
length; the last sequence stops after its literals).  XXH32 is the public
32-bit xxHash.

Parity: no lz4-java and no `.lz4` file exist in the build environment, so this
codec is pinned only to the public known answers of XXH32 and to hand-built LZ4
blocks (tests/test_smatio.py), not to a file written by BIDMat: "parity
unpinned" for the container layer.  The reader therefore compares only the 28
checksum bits every version of the writer stores and accepts the end of the
file in place of a missing end-block.

Pure Python: meant for the matrix files of tests and examples (reads about
8 MB/s, writes about 3 MB/s).
"""
import io
import struct

MAGIC = b"LZ4Block"
_HEADER = struct.Struct("<8sBiii")
_METHOD_RAW, _METHOD_LZ4 = 0x10, 0x20
_LEVEL_BASE = 10
_SEED = 0x9747B28C
_M32 = 0xFFFFFFFF
_P1, _P2, _P3, _P4, _P5 = 2654435761, 2246822519, 3266489917, 668265263, 374761393


def _rotl(x, r):
    return ((x << r) | (x >> (32 - r))) & _M32


def xxh32(data, seed=0):
    """32-bit xxHash of a bytes-like object."""
    data = bytes(data)
    n = len(data)
    i = 0
    if n >= 16:
        v1 = (seed + _P1 + _P2) & _M32
        v2 = (seed + _P2) & _M32
        v3 = seed & _M32
        v4 = (seed - _P1) & _M32
        words = struct.unpack_from("<%dI" % ((n // 16) * 4), data, 0)
        for j in range(0, len(words), 4):
            v1 = (_rotl((v1 + words[j] * _P2) & _M32, 13) * _P1) & _M32
            v2 = (_rotl((v2 + words[j + 1] * _P2) & _M32, 13) * _P1) & _M32
            v3 = (_rotl((v3 + words[j + 2] * _P2) & _M32, 13) * _P1) & _M32
            v4 = (_rotl((v4 + words[j + 3] * _P2) & _M32, 13) * _P1) & _M32
        i = (n // 16) * 16
        h = (_rotl(v1, 1) + _rotl(v2, 7) + _rotl(v3, 12) + _rotl(v4, 18)) & _M32
    else:
        h = (seed + _P5) & _M32
    h = (h + n) & _M32
    while i + 4 <= n:
        h = (_rotl((h + struct.unpack_from("<I", data, i)[0] * _P3) & _M32, 17) * _P4) & _M32
        i += 4
    while i < n:
        h = (_rotl((h + data[i] * _P5) & _M32, 11) * _P1) & _M32
        i += 1
    h ^= h >> 15
    h = (h * _P2) & _M32
    h ^= h >> 13
    h = (h * _P3) & _M32
    h ^= h >> 16
    return h


def decompress_block(src, original_length):
    """One LZ4 block -> bytes of exactly original_length."""
    src = bytes(src)
    out = bytearray()
    i, n = 0, len(src)
    while i < n:
        token = src[i]
        i += 1
        lit = token >> 4
        if lit == 15:
            while True:
                if i >= n:
                    raise ValueError("LZ4 block: literal length runs past the end")
                b = src[i]
                i += 1
                lit += b
                if b != 255:
                    break
        if i + lit > n:
            raise ValueError("LZ4 block: literals run past the end")
        out += src[i:i + lit]
        i += lit
        if i >= n:
            break                       # the last sequence has no match
        if i + 2 > n:
            raise ValueError("LZ4 block: truncated match offset")
        offset = src[i] | (src[i + 1] << 8)
        i += 2
        if offset == 0 or offset > len(out):
            raise ValueError("LZ4 block: match offset %d outside the %d bytes decoded so far" % (offset, len(out)))
        mlen = token & 15
        if mlen == 15:
            while True:
                if i >= n:
                    raise ValueError("LZ4 block: match length runs past the end")
                b = src[i]
                i += 1
                mlen += b
                if b != 255:
                    break
        mlen += 4
        start = len(out) - offset
        if offset >= mlen:
            out += out[start:start + mlen]
        else:                           # overlapping match: the pattern repeats
            pattern = bytes(out[start:])
            reps, rest = divmod(mlen, offset)
            out += pattern * reps + pattern[:rest]
    if len(out) != original_length:
        raise ValueError("LZ4 block: decoded %d bytes, the header says %d" % (len(out), original_length))
    return bytes(out)


def _put_length(out, extra):
    while extra >= 255:
        out.append(255)
        extra -= 255
    out.append(extra)


def compress_block(data):
    """Greedy LZ4 block compressor (4-byte hash matches, 64 KB window).  Obeys the end-of-block
    rules of the format: the last 5 bytes are literals and no match starts in the last 12."""
    data = bytes(data)
    n = len(data)
    out = bytearray()
    anchor = 0
    i = 0
    table = {}
    limit = n - 12
    while i < limit:
        key = data[i:i + 4]
        cand = table.get(key, -1)
        table[key] = i
        if cand < 0 or i - cand > 65535:
            i += 1
            continue
        mlen = 4
        mmax = n - 5 - i
        while mlen < mmax and data[cand + mlen] == data[i + mlen]:
            mlen += 1
        if mlen < 4 or mmax < 4:
            i += 1
            continue
        lit = i - anchor
        out.append((min(lit, 15) << 4) | min(mlen - 4, 15))
        if lit >= 15:
            _put_length(out, lit - 15)
        out += data[anchor:i]
        off = i - cand
        out.append(off & 255)
        out.append(off >> 8)
        if mlen - 4 >= 15:
            _put_length(out, mlen - 4 - 15)
        i += mlen
        anchor = i
    lit = n - anchor
    out.append(min(lit, 15) << 4)
    if lit >= 15:
        _put_length(out, lit - 15)
    out += data[anchor:]
    return bytes(out)


class LZ4BlockReader(io.RawIOBase):
    """File-like reader of an lz4-java block stream (what LZ4BlockInputStream reads)."""

    def __init__(self, raw, verify=True):
        self._raw, self._verify = raw, verify
        self._buf, self._pos, self._done = b"", 0, False

    def readable(self):
        return True

    def _next_block(self):
        head = self._raw.read(_HEADER.size)
        if len(head) == 0:
            self._done = True           # a stream cut after its last block: accepted
            return
        if len(head) != _HEADER.size:
            raise RuntimeError("lz4 block stream: truncated block header")
        magic, token, clen, olen, check = _HEADER.unpack(head)
        if magic != MAGIC:
            raise RuntimeError("lz4 block stream: bad magic %r (an LZ4 *frame* file is a different format)" % magic)
        method, level = token & 0xF0, token & 0x0F
        if (method not in (_METHOD_RAW, _METHOD_LZ4) or clen < 0 or olen < 0 or olen > (1 << (_LEVEL_BASE + level))
                or (method == _METHOD_RAW and clen != olen) or (olen == 0) != (clen == 0)):
            raise RuntimeError("lz4 block stream: corrupt block header")
        if olen == 0:
            self._done = True
            return
        payload = self._raw.read(clen)
        if len(payload) != clen:
            raise RuntimeError("lz4 block stream: truncated block")
        data = payload if method == _METHOD_RAW else decompress_block(payload, olen)
        if self._verify and ((xxh32(data, _SEED) ^ check) & 0x0FFFFFFF):
            raise RuntimeError("lz4 block stream: checksum mismatch")
        self._buf, self._pos = data, 0

    def read(self, size=-1):
        parts = []
        while size != 0:
            if self._pos >= len(self._buf):
                if self._done:
                    break
                self._next_block()
                continue
            take = len(self._buf) - self._pos if size < 0 else min(size, len(self._buf) - self._pos)
            parts.append(self._buf[self._pos:self._pos + take])
            self._pos += take
            if size > 0:
                size -= take
        return b"".join(parts)

    def close(self):
        if not self.closed:
            self._raw.close()
        super().close()


class LZ4BlockWriter(io.RawIOBase):
    """File-like writer of an lz4-java block stream with 64 KB blocks (the block size BIDMat
    asks for, HMat.scala:105-107); a block that does not shrink is stored raw."""

    def __init__(self, raw, block_size=1 << 16):
        level = max(0, (block_size - 1).bit_length() - _LEVEL_BASE)
        if (1 << (_LEVEL_BASE + level)) != block_size or level > 15:
            raise ValueError("block size must be a power of two between 1 KB and 32 MB")
        self._raw, self._size, self._level = raw, block_size, level
        self._pending = bytearray()

    def writable(self):
        return True

    def _emit(self, data):
        packed = compress_block(data)
        method = _METHOD_LZ4 if len(packed) < len(data) else _METHOD_RAW
        payload = packed if method == _METHOD_LZ4 else data
        check = xxh32(data, _SEED) & 0x0FFFFFFF
        self._raw.write(_HEADER.pack(MAGIC, method | self._level, len(payload), len(data), check))
        self._raw.write(payload)

    def write(self, b):
        self._pending += b
        while len(self._pending) >= self._size:
            self._emit(bytes(self._pending[:self._size]))
            del self._pending[:self._size]
        return len(b)

    def close(self):
        if not self.closed:
            if self._pending:
                self._emit(bytes(self._pending))
                self._pending = bytearray()
            self._raw.write(_HEADER.pack(MAGIC, _METHOD_RAW | self._level, 0, 0, 0))
            self._raw.close()
        super().close()
