from .engine import (CacheConfig, EngineBuilder, EngineConfig, EngineCore, EnginePresets, GenerationParams,  # noqa: F401
                     InferenceResponse, MetricsAggregator, RequestMetrics, SchedulerConfig, SOTAAsyncStreamEngine,
                     SOTAInferenceEngine, StreamChunk, create_openai_server, main, run_bench)
