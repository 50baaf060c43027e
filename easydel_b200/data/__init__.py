"""Data pipeline: sharded sources, transforms (tokenise, chat template, packing, mixing), loaders and writers."""

from .loader import IterableBatchLoader, PrefetchIterator, ShardedBatchLoader, build_loader
from .sources import (ArrowDataSource, CompositeDataSource, CsvDataSource, HuggingFaceDataSource, InMemorySource,
                      JsonDataSource, ParquetDataSource, ShardedDataSource, SourceState, TextDataSource,
                      create_source)
from .transforms import (ChatTemplateTransform, FilteredSource, FirstFitPacker, GreedyPacker, MappedSource,
                         MixtureSource, PackedShardedSource, PoolPacker, TokenizeTransform)
from .pipeline import DatasetConfig, Pipeline, PipelineConfig, TreeCache, save_source

AsyncDataLoader = ShardedBatchLoader

__all__ = [n for n in dir() if not n.startswith("_")]
