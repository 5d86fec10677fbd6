"""Local-filesystem stand-in for the ``megfile`` package (not installable offline): just the calls
the reference makes, mapped to ``os`` / ``open``."""
import os


def smart_open(path, mode="r", **kw):
    if any(m in mode for m in ("w", "a", "x")):
        d = os.path.dirname(str(path))
        if d:
            os.makedirs(d, exist_ok=True)
    kw.pop("s3_open_func", None)
    return open(path, mode, **{k: v for k, v in kw.items() if k in ("encoding", "newline", "buffering", "errors")})


def smart_exists(path):
    return os.path.exists(path)


def smart_path_join(*parts):
    return os.path.join(*[str(p) for p in parts])


def smart_makedirs(path, exist_ok=True):
    os.makedirs(path, exist_ok=exist_ok)


def smart_getsize(path):
    return os.path.getsize(path)


def smart_remove(path, missing_ok=True):
    try:
        os.remove(path)
    except FileNotFoundError:
        if not missing_ok:
            raise


def smart_listdir(path):
    return sorted(os.listdir(path))


def smart_isdir(path):
    return os.path.isdir(path)


def smart_glob(pattern):
    import glob

    return sorted(glob.glob(pattern))


def smart_rename(src, dst, overwrite=True):
    os.replace(src, dst)


def smart_copy(src, dst, **kw):
    import shutil

    shutil.copy(src, dst)


def smart_isfile(path):
    return os.path.isfile(path)


def smart_touch(path):
    open(path, "a").close()


def smart_unlink(path, missing_ok=True):
    smart_remove(path, missing_ok)
