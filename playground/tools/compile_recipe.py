"""Datasets configs that read a :class:`DataRecipe` of raw chat JSON files, and their compiled (pre-tokenised,
indexed-bin) form (reference ``playground/tools/compile_recipe.py``).

``CompilableDatasetsConfig`` templates every raw conversation on the fly; ``compile(path)`` writes each domain as
a compiled dataset under ``path/<domain>`` and returns the source text of the matching
``CompiledDatasetsConfig`` subclass; training from the compiled form gives the same samples, faster.

    python playground/tools/compile_recipe.py my_data_config.py:MyDatasetsConfig /data/compiled [--shards 8]
"""
from __future__ import annotations

import os

from steptronoss_b200.data.recipe import CompiledDataRecipe, DataRecipe
from steptronoss_b200.exp.sft import SFTDatasetsConfig
from steptronoss_b200.utils.logger import logger


class CompilableDatasetsConfig(SFTDatasetsConfig):
    def get_template(self):
        raise NotImplementedError

    def get_recipe(self) -> DataRecipe:
        raise NotImplementedError

    def get_dataset(self, files: list, template):
        from steptronoss_b200.data.datasets import StepChatJsonDataset

        return StepChatJsonDataset([getattr(f, "path", f) for f in files], template=template)

    def build_datasets(self) -> dict:
        recipe, template = self.get_recipe(), self.get_template()
        return {name: (self.get_dataset(files, template), recipe.epochs[name]) for name, files in recipe.domains.items()}

    def compile(self, compile_path: str, n_shards: int = 1) -> str:
        from steptronoss_b200.data.datasets import compile_dataset

        recipe, template = self.get_recipe(), self.get_template()
        compiled = {}
        for name, files in recipe.domains.items():
            out = os.path.join(compile_path, name)
            compile_dataset(self.get_dataset(files, template), out, n_shards=n_shards)
            compiled[name] = out
            logger.info(f"compiled domain {name} -> {out}")
        lines = ["from playground.tools.compile_recipe import CompiledDatasetsConfig",
                 "from steptronoss_b200.data.recipe import CompiledDataRecipe", "", "",
                 "class DatasetsConfig(CompiledDatasetsConfig):", "    compiled_recipe = CompiledDataRecipe(",
                 "        domains={"]
        lines += [f"            {n!r}: {p!r}," for n, p in compiled.items()]
        lines += ["        },", "        epochs={"]
        lines += [f"            {n!r}: {e}," for n, e in recipe.epochs.items()]
        lines += ["        },", "    )", ""]
        text = "\n".join(lines)
        logger.info("compiled recipe:\n" + text)
        return text


CompliableDatasetsConfig = CompilableDatasetsConfig  # the reference's spelling


class CompiledDatasetsConfig(SFTDatasetsConfig):
    compiled_recipe: CompiledDataRecipe

    def build_datasets(self) -> dict:
        from steptronoss_b200.data.datasets import CompiledDataset

        r = self.compiled_recipe
        return {name: (CompiledDataset(path), r.epochs[name]) for name, path in r.domains.items()}


def main(argv=None) -> int:
    import argparse

    from steptronoss_b200.config.mock_imports import get_object_from_file

    ap = argparse.ArgumentParser(description="Compile the raw recipe of a datasets config.")
    ap.add_argument("config", help="file.py:ClassName of a CompilableDatasetsConfig")
    ap.add_argument("out")
    ap.add_argument("--shards", type=int, default=1)
    a = ap.parse_args(argv)
    path, _, name = a.config.partition(":")
    cls = get_object_from_file(path, name or "DatasetsConfig")
    print(cls().compile(a.out, a.shards))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
