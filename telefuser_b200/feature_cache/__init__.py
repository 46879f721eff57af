from .base import BaseFeatureCache, NoOpCache, create_feature_cache

__all__ = ["BaseFeatureCache", "NoOpCache", "create_feature_cache"]
