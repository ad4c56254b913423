"""Ready-made patterns: expert-parallel MoE and KV-cache page migration.

Same names as the reference package (python/aboleth/patterns/__init__.py:1-22).
"""
from .kv_cache import KVCacheMigrationSpec, build_kv_cache_migration_pattern
from .kv_cache_transport import (CompiledKVCacheMigrationPlan, KVCacheLayoutContract,
                                 KVCachePhysicalization, compile_kv_cache_migration)
from .moe import MoEPatternSpec, build_moe_pattern

__all__ = [
    "CompiledKVCacheMigrationPlan", "KVCacheLayoutContract", "KVCacheMigrationSpec",
    "KVCachePhysicalization", "MoEPatternSpec", "build_kv_cache_migration_pattern",
    "build_moe_pattern", "compile_kv_cache_migration",
]
