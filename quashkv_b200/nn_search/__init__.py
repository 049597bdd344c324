from .index import QuashIndex

__all__ = ["QuashIndex"]
