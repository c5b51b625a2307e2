"""Model families. ``MODEL_CLASSES`` maps an HF ``model_type`` to its pipeline-chunk class."""


class _Lazy(dict):
    _paths = {
        "qwen3_moe": ("qwen3_moe", "Qwen3MoeModel"),
        "deepseek_v2": ("deepseek_v2", "DeepSeekV2Model"),
        "gpt_oss": ("gpt_oss", "GptOssModel"),
        "qwen3_5_moe_text": ("qwen35_moe", "Qwen35MoeModel"),
    }

    def __contains__(self, k):
        return k in self._paths

    def __getitem__(self, k):
        import importlib

        mod, cls = self._paths[k]
        return getattr(importlib.import_module(f"{__name__}.{mod}"), cls)

    def keys(self):
        return self._paths.keys()


MODEL_CLASSES = _Lazy()
