#!/usr/bin/env python3
"""
Convert a Bliss corpus to the zip layout that ``OggZipDataset`` reads: ``<name>/<name>.txt`` (a Python list of
``{"file", "seq_name", "text", "duration"}``) and one audio file per segment. Segments are cut out of the recordings with the
``soundfile`` package (wav / flac / ogg, whatever it can write; ``--format wav`` works with the standard library for wav input).
(reference: tools/bliss-to-ogg-zip.py, which shells out to ffmpeg)
"""

import argparse
import io
import os
import wave
import zipfile
import _setup_returnn_env  # noqa: F401
from _bliss import iter_bliss


def _cut_wav(path: str, start: float, end: float) -> bytes:
    with wave.open(path, "rb") as w:
        rate = w.getframerate()
        w.setpos(min(int(start * rate), w.getnframes()))
        n = max(0, min(int((end - start) * rate) if end > start else w.getnframes(), w.getnframes() - w.tell()))
        frames = w.readframes(n)
        buf = io.BytesIO()
        with wave.open(buf, "wb") as out:
            out.setnchannels(w.getnchannels())
            out.setsampwidth(w.getsampwidth())
            out.setframerate(rate)
            out.writeframes(frames)
        return buf.getvalue()


def _cut_soundfile(path: str, start: float, end: float, fmt: str) -> bytes:
    import soundfile

    info = soundfile.info(path)
    a = int(start * info.samplerate)
    b = int(end * info.samplerate) if end > start else info.frames
    data, rate = soundfile.read(path, start=a, stop=b)
    buf = io.BytesIO()
    soundfile.write(buf, data, rate, format=fmt.upper())
    return buf.getvalue()


def main():
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("bliss_filename")
    ap.add_argument("--output", required=True, help="output .zip")
    ap.add_argument("--format", default="ogg", help="audio format inside the zip (ogg, flac, wav)")
    ap.add_argument("--no-audio", action="store_true", help="only the text file (e.g. for a text-only dataset)")
    args = ap.parse_args()
    name = os.path.splitext(os.path.basename(args.output))[0]
    entries = []
    with zipfile.ZipFile(args.output, "w", zipfile.ZIP_STORED) as zf:
        for item in iter_bliss(args.bliss_filename):
            rel = "%s.%s" % (item.segment_name.replace("/", "_"), args.format)
            if not args.no_audio:
                assert item.recording_filename, "segment %s has no recording" % item.segment_name
                if args.format == "wav" and item.recording_filename.endswith(".wav"):
                    data = _cut_wav(item.recording_filename, item.start_time, item.end_time)
                else:
                    data = _cut_soundfile(item.recording_filename, item.start_time, item.end_time, args.format)
                zf.writestr("%s/%s" % (name, rel), data)
            entries.append({"file": rel, "seq_name": item.segment_name, "text": item.orth or "", "duration": item.delta_time})
        zf.writestr("%s.txt" % name, "[\n" + "".join("%r,\n" % e for e in entries) + "]\n")
    print("wrote %i segments to %s" % (len(entries), args.output))


if __name__ == "__main__":
    main()
