"""
Audio feature extraction on the host in plain numpy (reference: returnn/datasets/util/feature_extraction.py:10,
which calls librosa): ``raw``, ``log_mel_filterbank``, ``log_log_mel_filterbank``, ``db_mel_filterbank``,
``linear_spectrogram``, ``mfcc``; optional delta features, pre-emphasis, per-sequence normalisation, random permutation
of the audio (speed / tempo via resampling by linear interpolation).
"""

from __future__ import annotations
from typing import Any, Callable, Dict, Optional, Union
import numpy


def _hz_to_mel(f):
    return 2595.0 * numpy.log10(1.0 + numpy.asarray(f, dtype="float64") / 700.0)


def _mel_to_hz(m):
    return 700.0 * (10.0 ** (numpy.asarray(m, dtype="float64") / 2595.0) - 1.0)


def mel_filterbank_matrix(sample_rate: int, n_fft: int, n_mels: int, f_min: float = 0.0, f_max: Optional[float] = None) -> numpy.ndarray:
    """triangular filters, ``[n_fft // 2 + 1, n_mels]`` (HTK mel scale, unnormalised)"""
    f_max = f_max or sample_rate / 2.0
    mel_pts = numpy.linspace(_hz_to_mel(f_min), _hz_to_mel(f_max), n_mels + 2)
    hz_pts = _mel_to_hz(mel_pts)
    freqs = numpy.linspace(0.0, sample_rate / 2.0, n_fft // 2 + 1)
    fb = numpy.zeros((n_fft // 2 + 1, n_mels), dtype="float32")
    for m in range(n_mels):
        lo, ce, hi = hz_pts[m], hz_pts[m + 1], hz_pts[m + 2]
        up = (freqs - lo) / max(ce - lo, 1e-10)
        down = (hi - freqs) / max(hi - ce, 1e-10)
        fb[:, m] = numpy.maximum(0.0, numpy.minimum(up, down))
    return fb


def _frames(audio: numpy.ndarray, win: int, step: int, center: bool) -> numpy.ndarray:
    if center:
        audio = numpy.pad(audio, (win // 2, win // 2), mode="reflect" if len(audio) > win // 2 else "constant")
    if len(audio) < win:
        audio = numpy.pad(audio, (0, win - len(audio)))
    n = 1 + (len(audio) - win) // step
    idx = numpy.arange(win)[None, :] + step * numpy.arange(n)[:, None]
    return audio[idx]


def power_spectrogram(audio: numpy.ndarray, sample_rate: int, window_len: float, step_len: float, center: bool = True):
    """:return: ([frames, n_fft//2+1] power, n_fft)"""
    win = int(window_len * sample_rate)
    step = int(step_len * sample_rate)
    n_fft = 1 << (win - 1).bit_length()
    fr = _frames(audio.astype("float32"), win, step, center) * numpy.hanning(win + 1)[:-1].astype("float32")
    spec = numpy.fft.rfft(fr, n=n_fft, axis=1)
    return (spec.real ** 2 + spec.imag ** 2).astype("float32"), n_fft


def _dct2(x: numpy.ndarray, n_out: int) -> numpy.ndarray:
    n = x.shape[1]
    k = numpy.arange(n_out)[None, :]
    i = numpy.arange(n)[:, None]
    basis = numpy.cos(numpy.pi / n * (i + 0.5) * k) * numpy.sqrt(2.0 / n)
    basis[:, 0] *= numpy.sqrt(0.5)
    return (x @ basis).astype("float32")


def _deltas(feat: numpy.ndarray, width: int = 9) -> numpy.ndarray:
    half = width // 2
    padded = numpy.pad(feat, ((half, half), (0, 0)), mode="edge")
    num = sum(k * (padded[half + k: half + k + len(feat)] - padded[half - k: half - k + len(feat)]) for k in range(1, half + 1))
    return (num / (2.0 * sum(k * k for k in range(1, half + 1)))).astype("float32")


class ExtractAudioFeatures:
    """callable feature pipeline configured like the reference's class of the same name"""

    def __init__(self, window_len: float = 0.025, step_len: float = 0.010, num_feature_filters: Optional[int] = None, with_delta: Union[bool, int] = False,
                 norm_mean: Optional[Union[str, float, numpy.ndarray]] = None, norm_std_dev: Optional[Union[str, float, numpy.ndarray]] = None,
                 features: Union[str, Callable] = "mfcc", feature_options: Optional[Dict[str, Any]] = None, random_permute: Optional[Union[bool, Dict[str, Any]]] = None,
                 random_state: Optional[numpy.random.RandomState] = None, raw_ogg_opts=None, pre_process: Optional[Callable] = None,
                 post_process: Optional[Callable] = None, sample_rate: Optional[int] = None, num_channels: Optional[int] = None, peak_normalization: bool = True,
                 preemphasis: Optional[float] = None, join_frames: Optional[int] = None):
        self.window_len, self.step_len = window_len, step_len
        self.features = features
        if num_feature_filters is None:
            num_feature_filters = {"mfcc": 40, "log_mel_filterbank": 80, "log_log_mel_filterbank": 80, "db_mel_filterbank": 80, "raw": 1}.get(
                features if isinstance(features, str) else "", 1)
        self.num_feature_filters = num_feature_filters
        self.with_delta = int(with_delta) if not isinstance(with_delta, bool) else (1 if with_delta else 0)
        self.norm_mean = self._load(norm_mean)
        self.norm_std_dev = self._load(norm_std_dev)
        self.feature_options = feature_options or {}
        self.random_permute = {"rnd_scale_lower": 1.0, "rnd_scale_upper": 1.0} if random_permute is True else (random_permute or None)
        self.random_state = random_state or numpy.random.RandomState(1)
        self.pre_process, self.post_process = pre_process, post_process
        self.sample_rate = sample_rate
        self.num_channels = num_channels
        self.peak_normalization = peak_normalization
        self.preemphasis = preemphasis
        self.join_frames = join_frames

    @staticmethod
    def _load(v):
        if v is None or isinstance(v, (int, float)):
            return v
        if isinstance(v, str):
            if v == "per_seq":
                return v
            return numpy.loadtxt(v).astype("float32")
        return numpy.asarray(v, dtype="float32")

    def get_feature_dimension(self) -> int:
        """output feature dim"""
        return (self.with_delta + 1) * self.num_feature_filters * (self.num_channels or 1) * (self.join_frames or 1)

    def get_audio_features(self, audio: numpy.ndarray, sample_rate: int, seq_name: Optional[str] = None) -> numpy.ndarray:
        """:param audio: [samples] or [samples, channels]; :return: [frames, feature_dim] float32"""
        if self.sample_rate is not None:
            assert sample_rate == self.sample_rate, "%s: audio has sample rate %i, expected %i" % (seq_name, sample_rate, self.sample_rate)
        audio = numpy.asarray(audio, dtype="float32")
        if audio.ndim == 2:
            chans = [self.get_audio_features(audio[:, c], sample_rate, seq_name) for c in range(audio.shape[1])]
            n = min(len(c) for c in chans)
            return numpy.concatenate([c[:n] for c in chans], axis=1)
        if self.pre_process:
            audio = self.pre_process(audio=audio, sample_rate=sample_rate, random_state=self.random_state)
        if self.random_permute:
            audio = _random_permute_audio(audio, sample_rate, self.random_permute, self.random_state)
        if self.peak_normalization and len(audio):
            peak = numpy.max(numpy.abs(audio))
            if peak > 0:
                audio = audio / peak
        if self.preemphasis:
            audio = numpy.concatenate([audio[:1], audio[1:] - self.preemphasis * audio[:-1]]).astype("float32")
        f = self.features
        if callable(f):
            feat = f(audio=audio, sample_rate=sample_rate, window_len=self.window_len, step_len=self.step_len, num_feature_filters=self.num_feature_filters,
                     random_state=self.random_state, **self.feature_options)
        elif f == "raw":
            feat = audio[:, None]
        else:
            power, n_fft = power_spectrogram(audio, sample_rate, self.window_len, self.step_len, center=self.feature_options.get("center", True))
            if f == "linear_spectrogram":
                feat = numpy.sqrt(power)[:, : self.num_feature_filters]
            else:
                n_mels = self.num_feature_filters if f != "mfcc" else self.feature_options.get("n_mels", 128)
                mel = power @ mel_filterbank_matrix(sample_rate, n_fft, n_mels, self.feature_options.get("fmin", 0.0), self.feature_options.get("fmax"))
                if f == "log_mel_filterbank":
                    feat = numpy.log(numpy.maximum(mel, 1e-10))
                elif f == "log_log_mel_filterbank":
                    feat = numpy.log(numpy.log(numpy.maximum(mel, 1e-10) + 1.0) + 1e-10)
                elif f == "db_mel_filterbank":
                    db = 10.0 * numpy.log10(numpy.maximum(mel, 1e-10))
                    feat = numpy.maximum(db, db.max() - self.feature_options.get("top_db", 80.0))
                elif f == "mfcc":
                    feat = _dct2(10.0 * numpy.log10(numpy.maximum(mel, 1e-10)), self.num_feature_filters)
                else:
                    raise ValueError("unknown feature type %r" % (f,))
        feat = feat.astype("float32")
        if self.with_delta:
            parts, cur = [feat], feat
            for _ in range(self.with_delta):
                cur = _deltas(cur)
                parts.append(cur)
            feat = numpy.concatenate(parts, axis=1)
        if isinstance(self.norm_mean, str) and self.norm_mean == "per_seq":
            feat = feat - feat.mean(axis=0, keepdims=True)
        elif self.norm_mean is not None:
            feat = feat - self.norm_mean
        if isinstance(self.norm_std_dev, str) and self.norm_std_dev == "per_seq":
            feat = feat / numpy.maximum(feat.std(axis=0, keepdims=True), 1e-2)
        elif self.norm_std_dev is not None:
            feat = feat / self.norm_std_dev
        if self.join_frames:
            pad = (-len(feat)) % self.join_frames
            if pad:
                feat = numpy.concatenate([feat, numpy.zeros((pad, feat.shape[1]), "float32")])
            feat = feat.reshape(len(feat) // self.join_frames, -1)
        if self.post_process:
            feat = self.post_process(feat, seq_name=seq_name)
        return feat.astype("float32")


def _random_permute_audio(audio: numpy.ndarray, sample_rate: int, opts: Dict[str, Any], rnd: numpy.random.RandomState) -> numpy.ndarray:
    """random tempo change by resampling with a random factor in [rnd_scale_lower, rnd_scale_upper], random gain"""
    lo, hi = opts.get("rnd_scale_lower", 0.9), opts.get("rnd_scale_upper", 1.1)
    factor = rnd.uniform(lo, hi)
    if abs(factor - 1.0) > 1e-6 and len(audio) > 1:
        n_new = max(int(round(len(audio) / factor)), 1)
        audio = numpy.interp(numpy.linspace(0, len(audio) - 1, n_new), numpy.arange(len(audio)), audio).astype("float32")
    if opts.get("rnd_gain"):
        audio = audio * float(10.0 ** (rnd.uniform(-opts["rnd_gain"], opts["rnd_gain"]) / 20.0))
    return audio
