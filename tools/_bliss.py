"""Streaming reader for Bliss corpus XML files (optionally gzipped), shared by the bliss-* tools."""

import gzip
import xml.etree.ElementTree as ElementTree
from typing import Iterator, NamedTuple, Optional


class BlissItem(NamedTuple):
    """one segment"""

    segment_name: str
    recording_filename: Optional[str]
    start_time: float
    end_time: float
    orth: Optional[str]
    speaker_name: Optional[str]

    @property
    def delta_time(self) -> float:
        return self.end_time - self.start_time


def iter_bliss(filename: str) -> Iterator[BlissItem]:
    """yields the segments of a corpus file, following <include file=...> of sub-corpora relative to the file"""
    import os

    f = gzip.open(filename, "rb") if filename.endswith(".gz") else open(filename, "rb")
    name_stack, rec_stack = [], []
    elem_stack = []
    for event, elem in ElementTree.iterparse(f, events=("start", "end")):
        if event == "start":
            elem_stack.append(elem)
            if elem.tag in ("corpus", "subcorpus", "recording"):
                name_stack.append(elem.attrib.get("name", ""))
            if elem.tag == "recording":
                rec_stack.append(elem.attrib.get("audio"))
        else:
            elem_stack.pop()
            if elem.tag == "include":
                inc = os.path.join(os.path.dirname(filename), elem.attrib["file"])
                for item in iter_bliss(inc):
                    yield item
            elif elem.tag == "segment":
                orth_el = elem.find("orth")
                spk_el = elem.find("speaker")
                seg_name = "/".join([n for n in name_stack if n] + [elem.attrib.get("name", "")])
                yield BlissItem(segment_name=seg_name, recording_filename=rec_stack[-1] if rec_stack else None,
                                start_time=float(elem.attrib.get("start", 0.0)), end_time=float(elem.attrib.get("end", 0.0)),
                                orth=" ".join(orth_el.text.split()) if orth_el is not None and orth_el.text else None,
                                speaker_name=spk_el.attrib.get("name") if spk_el is not None else None)
                elem.clear()
            elif elem.tag in ("corpus", "subcorpus", "recording"):
                name_stack.pop()
                if elem.tag == "recording":
                    rec_stack.pop()
                elem.clear()
    f.close()
