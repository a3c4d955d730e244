"""``EvaluationTools`` (``deeplearning4j-core/.../evaluation/EvaluationTools.java``): standalone HTML reports
(ROC / precision-recall charts as inline SVG, calibration tables) for evaluation objects."""
from __future__ import annotations

import html


def _svg_curve(xs, ys, title, xlabel, ylabel, w=420, h=320, pad=40):
    pts = " ".join(f"{pad + x * (w - 2 * pad):.1f},{h - pad - y * (h - 2 * pad):.1f}" for x, y in zip(xs, ys))
    return (f'<svg xmlns="http://www.w3.org/2000/svg" width="{w}" height="{h}"><text x="{w / 2}" y="16" text-anchor="middle">{html.escape(title)}</text>'
            f'<rect x="{pad}" y="{pad}" width="{w - 2 * pad}" height="{h - 2 * pad}" fill="none" stroke="#888"/>'
            f'<polyline fill="none" stroke="#1f77b4" stroke-width="2" points="{pts}"/>'
            f'<text x="{w / 2}" y="{h - 8}" text-anchor="middle">{html.escape(xlabel)}</text>'
            f'<text x="12" y="{h / 2}" transform="rotate(-90 12 {h / 2})" text-anchor="middle">{html.escape(ylabel)}</text></svg>')


class EvaluationTools:
    @staticmethod
    def rocChartToHtml(roc, classNames=None):
        from .roc import ROC
        parts = ["<html><head><meta charset='utf-8'><title>ROC</title></head><body>"]
        rocs = [roc] if isinstance(roc, ROC) else list(roc.underlying or [])
        for i, r in enumerate(rocs):
            name = classNames[i] if classNames else (f"class {i}" if len(rocs) > 1 else "")
            c, pr = r.getRocCurve(), r.getPrecisionRecallCurve()
            parts.append(f"<h3>{html.escape(name)} AUC={r.calculateAUC():.4f} AUPRC={r.calculateAUCPR():.4f}</h3>")
            parts.append(_svg_curve(c.getX(), c.getY(), "ROC", "False positive rate", "True positive rate"))
            parts.append(_svg_curve(pr.getX(), pr.getY(), "Precision-Recall", "Recall", "Precision"))
        parts.append("</body></html>")
        return "".join(parts)

    @staticmethod
    def exportRocChartsToHtmlFile(roc, path, classNames=None):
        with open(path, "w") as f:
            f.write(EvaluationTools.rocChartToHtml(roc, classNames))

    @staticmethod
    def evaluationCalibrationToHtml(ec):
        parts = ["<html><body><h2>Calibration</h2>"]
        n = 0 if ec.rCounts is None else ec.rCounts.shape[0]
        for c in range(n):
            d = ec.getReliabilityDiagram(c)
            parts.append(_svg_curve(d["meanPredictedValueX"], d["fractionPositivesY"], d["title"], "Mean predicted value", "Fraction of positives"))
        parts.append("</body></html>")
        return "".join(parts)

    @staticmethod
    def exportevaluationCalibrationToHtmlFile(ec, path):
        with open(path, "w") as f:
            f.write(EvaluationTools.evaluationCalibrationToHtml(ec))
