"""Start-up helpers under the names of the reference's ``initialize.py`` (:13-87): seeding and the set-up of the
group that keeps tied input / output embeddings of a multi-token-prediction model in step across pipeline stages."""
from __future__ import annotations

from .parallel.embedding_sync import sync_shared_embeddings
from .parallel.state import _set_rng_seed, set_mpu_random_seed  # noqa: F401  (re-exported)


def set_random_seed(seed: int) -> None:
    """Seed python, numpy and torch (and the current GPU) of this process; no model-parallel streams."""
    _set_rng_seed(int(seed))


def mtp_initialize(models) -> list:
    """Build the ``EMB_SYNC`` groups over the pipeline stages that hold a copy of the token embedding and copy the
    first stage's weights to the others.  Returns the rows of the new family."""
    return sync_shared_embeddings(models)
