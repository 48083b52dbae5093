from .backend import (  # noqa: F401
    MAX_KV_SPLITS,
    AttnBackend,
    DecodeMetadata,
    PrefillMetadata,
    compute_num_kv_splits,
)
