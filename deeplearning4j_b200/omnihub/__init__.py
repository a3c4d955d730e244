"""Model hub (``omnihub``): resolve a pretrained model by framework and name in the local cache, download it when missing, convert
models of other frameworks into this framework's formats, and expose the zoo as ``Pretrained.samediff().resnet18()`` style
namespaces.

Reference: ``omnihub/src/main/java/org/eclipse/deeplearning4j/omnihub`` (``OmniHubUtils.java:53-150`` download + load,
``Framework.java`` input / output frameworks, ``BootstrapFromLocal.java:45-130`` conversion of a local model folder,
``ModelNamespaceGenerator.java`` + ``models/{Pretrained,SameDiffModels,Dl4jModels}.java`` generated namespaces).

Layout: ``$OMNIHUB_HOME`` (default ``~/.omnihub``) holds one folder per framework (lower case) with the model files; the hub URL
(``$OMNIHUB_URL``) serves the same layout.  Any URL scheme that ``urllib`` opens works, ``file://`` included, which is how the
download path is exercised without a network."""
from __future__ import annotations

import enum
import json
import os
import shutil
import urllib.request


class Framework(enum.Enum):
    SAMEDIFF = 0
    PYTORCH = 1
    TENSORFLOW = 2
    KERAS = 3
    DL4J = 4
    ONNX = 5
    HUGGINGFACE = 6

    def frameworkIndex(self): return self.value

    @staticmethod
    def isInput(f):
        """Frameworks whose files are converted (``Framework.java:42-52``)."""
        return f in (Framework.TENSORFLOW, Framework.KERAS, Framework.PYTORCH, Framework.ONNX)

    @staticmethod
    def isOutput(f): return not Framework.isInput(f)

    @staticmethod
    def outputFrameworkFor(f):
        if not Framework.isInput(f):
            raise ValueError(f"{f.name} is not an input framework")
        return Framework.SAMEDIFF if f in (Framework.ONNX, Framework.PYTORCH, Framework.TENSORFLOW) else Framework.DL4J

    @staticmethod
    def fromString(name):
        return Framework[name.upper()]


class OmnihubConfig:
    DEFAULT_OMNIHUB_URL = "https://raw.githubusercontent.com/KonduitAI/omnihub-zoo/main"

    @staticmethod
    def getOmnihubHome():
        d = os.environ.get("OMNIHUB_HOME", os.path.join(os.path.expanduser("~"), ".omnihub"))
        os.makedirs(d, exist_ok=True)
        return d

    @staticmethod
    def getOmnihubUrl():
        return os.environ.get("OMNIHUB_URL", OmnihubConfig.DEFAULT_OMNIHUB_URL).rstrip("/")


class OmniHubUtils:
    FRAMEWORKS = tuple(f.name.lower() for f in Framework)
    CHUNK = 1 << 20

    getCacheDir = staticmethod(OmnihubConfig.getOmnihubHome)

    @staticmethod
    def modelPath(framework, fileName):
        framework = framework.name.lower() if isinstance(framework, Framework) else str(framework).lower()
        if framework not in OmniHubUtils.FRAMEWORKS:
            raise ValueError(f"unknown framework '{framework}' (expected one of {OmniHubUtils.FRAMEWORKS})")
        return os.path.join(OmnihubConfig.getOmnihubHome(), framework, fileName)

    @staticmethod
    def downloadAndLoadFromZoo(framework, fileName, forceDownload=False, progress=None):
        """Path of the cached file, fetched from ``<hub url>/<framework>/<fileName>`` first when it is missing or ``forceDownload``.
        The download goes to a ``.part`` file and is renamed when complete, so an interrupted transfer never looks like a model;
        ``progress(bytesSoFar, totalOrNone)`` is called per chunk (``ProgressInputStream``)."""
        path = OmniHubUtils.modelPath(framework, fileName)
        if os.path.exists(path) and not forceDownload:
            return path
        fw = os.path.basename(os.path.dirname(path))
        url = f"{OmnihubConfig.getOmnihubUrl()}/{fw}/{fileName}"
        os.makedirs(os.path.dirname(path), exist_ok=True)
        part = path + ".part"
        try:
            with urllib.request.urlopen(url, timeout=60) as src, open(part, "wb") as dst:
                total = src.headers.get("Content-Length") if getattr(src, "headers", None) is not None else None
                total = int(total) if total else None
                done = 0
                while True:
                    chunk = src.read(OmniHubUtils.CHUNK)
                    if not chunk:
                        break
                    dst.write(chunk)
                    done += len(chunk)
                    if progress is not None:
                        progress(done, total)
            if total is not None and done != total:
                raise IOError(f"short download: {done} of {total} bytes")
            os.replace(part, path)
        except Exception as e:
            if os.path.exists(part):
                os.remove(part)
            raise IOError(f"model '{fileName}' is not in the local cache and could not be fetched from {url} ({e}); "
                          f"place it at {path}") from e
        return path

    @staticmethod
    def loadSameDiffModel(fileName, forceDownload=False):
        from ..samediff import SameDiff
        path = OmniHubUtils.downloadAndLoadFromZoo("samediff", fileName, forceDownload)
        return SameDiff.fromFlatFile(path) if path.endswith(".fb") else SameDiff.load(path)

    @staticmethod
    def loadNetwork(fileName, forceDownload=False):
        from ..nn import ModelGuesser
        return ModelGuesser.loadModelGuess(OmniHubUtils.downloadAndLoadFromZoo("dl4j", fileName, forceDownload))

    loadCompGraph = loadNetwork

    @staticmethod
    def loadForeign(framework, fileName, forceDownload=False):
        """ONNX / TensorFlow / TFLite / Keras files through the importers."""
        path = OmniHubUtils.downloadAndLoadFromZoo(framework, fileName, forceDownload)
        return BootstrapFromLocal.importModel(Framework.fromString(str(framework)) if not isinstance(framework, Framework) else framework, path)


class BootstrapFromLocal:
    """Converts every model found under ``<home>/<input framework>/`` into the output framework's format beside the others
    (``BootstrapFromLocal.java:45-130``): ONNX / TensorFlow / TFLite files become SameDiff ``.fb`` files under ``samediff/``, Keras
    models become DL4J zips under ``dl4j/``."""

    EXTENSIONS = {Framework.ONNX: (".onnx",), Framework.TENSORFLOW: (".pb", ".tflite"), Framework.KERAS: (".h5", ".json", ".keras")}

    @staticmethod
    def importModel(framework, path):
        from .. import importers
        if framework == Framework.ONNX:
            return importers.importOnnx(path)
        if framework == Framework.TENSORFLOW:
            return importers.importTFLite(path) if path.endswith(".tflite") else importers.importFrozenTF(path)
        if framework == Framework.KERAS:
            return importers.KerasModelImport.importKerasModelAndWeights(path)
        raise ValueError(f"no importer for framework '{framework.name}' (PyTorch and Hugging Face models are exported to ONNX first)")

    @staticmethod
    def convert(framework, path, home=None):
        """One model; returns the path written."""
        from ..nn import ModelSerializer
        home = home or OmnihubConfig.getOmnihubHome()
        out_fw = Framework.outputFrameworkFor(framework)
        stem = os.path.splitext(os.path.basename(path))[0]
        model = BootstrapFromLocal.importModel(framework, path)
        out_dir = os.path.join(home, out_fw.name.lower())
        os.makedirs(out_dir, exist_ok=True)
        if out_fw == Framework.SAMEDIFF:
            out = os.path.join(out_dir, stem + ".fb")
            model.asFlatFile(out)
        else:
            out = os.path.join(out_dir, stem + ".zip")
            ModelSerializer.writeModel(model, out, True)
        return out

    @staticmethod
    def run(home=None, onError="collect"):
        """All input-framework folders of ``home``; returns ``{source path: output path or the exception}``."""
        home = home or OmnihubConfig.getOmnihubHome()
        results = {}
        for fw, exts in BootstrapFromLocal.EXTENSIONS.items():
            d = os.path.join(home, fw.name.lower())
            if not os.path.isdir(d):
                continue
            for name in sorted(os.listdir(d)):
                if not name.endswith(exts):
                    continue
                src = os.path.join(d, name)
                try:
                    results[src] = BootstrapFromLocal.convert(fw, src, home)
                except Exception as e:                    # one unsupported model does not stop the rest
                    if onError != "collect":
                        raise
                    results[src] = e
        return results

    @staticmethod
    def main(argv=None):
        import argparse
        ap = argparse.ArgumentParser(description="convert the models under an omnihub folder")
        ap.add_argument("--home", default=None)
        a = ap.parse_args(argv)
        for src, out in BootstrapFromLocal.run(a.home).items():
            print(f"{src} -> {out}")


class ModelNamespace:
    """One framework's models as methods: ``ns.resnet18(forceDownload=False)`` loads ``resnet18.<ext>`` of that framework.  The
    model list comes from ``<home>/<framework>/index.json`` (``{"models": [{"name": ..., "file": ...}]}``, also fetched from the hub)
    or, without an index, from the files already in the cache (``ModelNamespaceGenerator.java`` builds the same list into source)."""

    def __init__(self, framework):
        self.framework = framework

    def _index(self):
        home = os.path.join(OmnihubConfig.getOmnihubHome(), self.framework.name.lower())
        idx = os.path.join(home, "index.json")
        if os.path.exists(idx):
            with open(idx) as f:
                return {m["name"]: m["file"] for m in json.load(f)["models"]}
        if os.path.isdir(home):
            return {_method_name(os.path.splitext(n)[0]): n for n in sorted(os.listdir(home)) if not n.endswith((".part", ".json"))}
        return {}

    def models(self):
        return sorted(self._index())

    def load(self, name, forceDownload=False):
        idx = self._index()
        if name not in idx:
            raise KeyError(f"no model '{name}' in the {self.framework.name.lower()} namespace (known: {sorted(idx)})")
        if self.framework == Framework.SAMEDIFF:
            return OmniHubUtils.loadSameDiffModel(idx[name], forceDownload)
        if self.framework == Framework.DL4J:
            return OmniHubUtils.loadNetwork(idx[name], forceDownload)
        return OmniHubUtils.loadForeign(self.framework, idx[name], forceDownload)

    def __getattr__(self, name):
        if name.startswith("_"):
            raise AttributeError(name)
        return lambda forceDownload=False: self.load(name, forceDownload)

    def __dir__(self):
        return sorted(set(super().__dir__()) | set(self._index()))


def _method_name(stem):
    """File stem -> method name the way the namespace generator does it: camel case over ``-`` / ``_`` / ``.`` separators."""
    parts = [p for p in stem.replace("-", "_").replace(".", "_").split("_") if p]
    if not parts:
        return stem
    return parts[0][0].lower() + parts[0][1:] + "".join(p[0].upper() + p[1:] for p in parts[1:])


class Pretrained:
    @staticmethod
    def samediff(): return ModelNamespace(Framework.SAMEDIFF)

    @staticmethod
    def dl4j(): return ModelNamespace(Framework.DL4J)

    @staticmethod
    def of(framework): return ModelNamespace(framework if isinstance(framework, Framework) else Framework.fromString(framework))


class ModelNamespaceGenerator:
    """Writes a namespace as source (one method per model), the form in which the reference ships ``SameDiffModels`` / ``Dl4jModels``."""

    @staticmethod
    def generate(framework, outPath=None):
        ns = ModelNamespace(framework)
        cls = {Framework.SAMEDIFF: "SameDiffModels", Framework.DL4J: "Dl4jModels"}.get(framework, framework.name.capitalize() + "Models")
        loader = {Framework.SAMEDIFF: "loadSameDiffModel", Framework.DL4J: "loadNetwork"}.get(framework)
        lines = ["from deeplearning4j_b200.omnihub import OmniHubUtils", "", "", f"class {cls}:"]
        idx = ns._index()
        if not idx:
            lines.append("    pass")
        for name, file in sorted(idx.items()):
            call = (f"OmniHubUtils.{loader}({file!r}, forceDownload)" if loader
                    else f"OmniHubUtils.loadForeign({framework.name.lower()!r}, {file!r}, forceDownload)")
            lines += [f"    def {name}(self, forceDownload=False):", f"        return {call}", ""]
        src = "\n".join(lines).rstrip() + "\n"
        if outPath:
            with open(outPath, "w") as f:
                f.write(src)
        return src


def clearCache(framework=None):
    """Removes the cached files of one framework (or all)."""
    home = OmnihubConfig.getOmnihubHome()
    for fw in ([framework] if framework else list(Framework)):
        d = os.path.join(home, fw.name.lower())
        if os.path.isdir(d):
            shutil.rmtree(d)
