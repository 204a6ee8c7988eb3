"""Content hash of everything the native library is built from (standard library only).

``build.py`` stores the hash beside the objects it compiled; ``_extension.py`` compares it before
loading, so that a library left over from older sources is reported instead of being loaded.
"""
import hashlib
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
CSRC = PACKAGE_DIR / "csrc"
INCLUDE = PACKAGE_DIR.parent / "include"
BUILD_DIR = PACKAGE_DIR / "build"
STAMP = BUILD_DIR / "fingerprint"
DEFINES = BUILD_DIR / "defines"


def source_fingerprint(flags, defines):
    digest = hashlib.sha256()
    sources = list(CSRC.glob("*")) + list(INCLUDE.glob("*.h")) + [PACKAGE_DIR / "build.py"]
    for path in sorted(sources):
        if path.is_file():
            digest.update(path.name.encode())
            digest.update(path.read_bytes())
    digest.update(repr((tuple(flags), tuple(defines))).encode())
    return digest.hexdigest()


def recorded_build():
    """``(fingerprint, flags, defines)`` of the last build in this tree, or None."""
    if not STAMP.is_file():
        return None
    if not DEFINES.is_file():
        return "", (), ()  # a stamp from before the flags were recorded: never matches
    lines = DEFINES.read_text().splitlines()
    if not lines:
        return None
    flags = tuple(lines[0].split("\t")) if lines[0] else ()
    defines = tuple(line for line in lines[1:] if line)
    return STAMP.read_text().strip(), flags, defines
