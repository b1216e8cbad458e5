from turboquant_b200.compressors import TurboQuantCompressorMSE, TurboQuantCompressorV2  # noqa: F401
