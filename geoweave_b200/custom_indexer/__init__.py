"""Drop-in for ``easyvolcap.utils.custom_indexer`` (reference ``__init__.py:1-13``)."""
from .sparse_topk_indexer import sparse_topk_indexer_func, sparse_topk_indexer_inference_func  # noqa: F401


def sparse_indexer_kl_loss(*args, **kwargs):
    raise NotImplementedError("the indexer KL loss is a training loss of the reference and is not part of this "
                              "inference library")


__all__ = ["sparse_topk_indexer_func", "sparse_topk_indexer_inference_func", "sparse_indexer_kl_loss"]
