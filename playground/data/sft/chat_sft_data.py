"""Chat SFT data from StepChat-style JSON files (reference
``playground/data/sft/oss260312/step_sft_data_config0311*.py``): a recipe of domains, templated with the
experiment tokenizer's chat template (assistant turns after the last user turn carry the loss), packed to the
trainer's sequence length.

Set ``STB200_SFT_DATA`` to a JSON file (or a comma list) of ``{"conversations": [...]}`` records and
``STB200_TOKENIZER`` to a HF tokenizer directory, or subclass ``ChatDatasetsConfig`` and override ``files`` /
``tokenizer_path``.  ``CompiledChatSFTDataConfig`` reads the compiled form written by
``ChatDatasetsConfig().compile(path)``.
"""
import os

from playground.tools.compile_recipe import CompilableDatasetsConfig, CompiledDatasetsConfig
from steptronoss_b200.data.recipe import CompiledDataRecipe, DataRecipe, DataSourceFile
from steptronoss_b200.exp.sft import SFTDataConfig


class ChatDatasetsConfig(CompilableDatasetsConfig):
    files: dict = {}
    """domain -> list of JSON paths; empty: the files named by ``STB200_SFT_DATA`` as one domain ``general``"""
    epochs: dict = {}
    tokenizer_path: str | None = None
    system_prompt: str | None = None

    def get_recipe(self) -> DataRecipe:
        files = dict(self.files)
        if not files:
            env = os.environ.get("STB200_SFT_DATA", "")
            if not env:
                raise ValueError("no SFT data: set ChatDatasetsConfig.files or the STB200_SFT_DATA variable")
            files = {"general": [p for p in env.split(",") if p]}
        domains = {d: [f if isinstance(f, DataSourceFile) else DataSourceFile(f) for f in fs] for d, fs in files.items()}
        return DataRecipe(domains=domains, epochs={d: self.epochs.get(d, 1) for d in domains})

    def get_template(self):
        from steptronoss_b200.data.chat_template import HuggingFaceTemplate
        from steptronoss_b200.tokenizer.hf_compat_tokenizer import HFCompatTokenizer

        path = self.tokenizer_path or os.environ.get("STB200_TOKENIZER")
        if not path:
            raise ValueError("no tokenizer: set ChatDatasetsConfig.tokenizer_path or the STB200_TOKENIZER variable")
        return HuggingFaceTemplate(HFCompatTokenizer.from_pretrained(path), self.system_prompt)


class ChatSFTDataConfig(SFTDataConfig):
    dataset_cfg = ChatDatasetsConfig
    oversize_policy = "drop"
    dataset_sampling = "sequential"
    num_workers = 16


class CompiledChatDatasetsConfig(CompiledDatasetsConfig):
    def __init__(self):
        super().__init__()
        root = os.environ.get("STB200_SFT_COMPILED", "")
        if root:
            self.compiled_recipe = CompiledDataRecipe(domains={"general": os.path.join(root, "general")},
                                                      epochs={"general": 1})


class CompiledChatSFTDataConfig(ChatSFTDataConfig):
    dataset_cfg = CompiledChatDatasetsConfig
