from .hashing import extend_hashes, page_hash, page_hashes  # noqa: F401
from .manager import CacheManager, OutOfPages, Sequence  # noqa: F401
from .pages import PagePool  # noqa: F401
