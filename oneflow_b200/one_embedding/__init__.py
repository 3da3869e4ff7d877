"""``flow.one_embedding``: large-scale embedding tables sharded over the ranks (see embedding.py)."""
from .embedding import (Embedding, Ftrl, MultiTableEmbedding, MultiTableMultiColumnEmbedding, Optimizer, SmartDecayAdam,  # noqa: F401
                        make_cached_host_mem_store_options, make_cached_ssd_store_options, make_column_options,
                        make_constant_initializer, make_device_mem_store_options, make_normal_initializer, make_table,
                        make_table_options, make_uniform_initializer, make_trunc_normal_initializer, PersistentTableReader,
                        PersistentTableWriter, make_persistent_table_reader, make_persistent_table_writer)
from .ops import OneEmbeddingHandler  # noqa: F401,E402
