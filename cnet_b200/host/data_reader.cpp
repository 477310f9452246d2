#include "data_reader.h"

#include <algorithm>
#include <fstream>
#include <random>

namespace cnet_b200 {

void BatchedDataReader::shuffle(unsigned seed) {
	std::mt19937 rng(seed);
	std::shuffle(samples_.begin(), samples_.end(), rng);
}

InputBatch BatchedDataReader::nextBatch(int batch_size) {
	InputBatch batch(batch_size, sample_dim_);
	if (samples_.empty()) return batch;
	for (int i = 0; i < batch_size; ++i) {
		batch.add(samples_[current_].data, samples_[current_].label);
		current_ = (current_ + 1) % samples_.size();
	}
	return batch;
}

bool BatchedDataReader::nextBatchInto(int batch_size, float* re, float* im, int* labels) {
	if (samples_.empty() || batch_size <= 0 || !re || !im || !labels) return false;
	for (int i = 0; i < batch_size; ++i) {
		const Record& r = samples_[current_];
		float* pr = re + (size_t) i * sample_dim_;
		float* pi = im + (size_t) i * sample_dim_;
		const int n = std::min<int>(sample_dim_, (int) r.data.size());
		for (int k = 0; k < n; ++k) { pr[k] = r.data[k].real(); pi[k] = r.data[k].imag(); }
		for (int k = n; k < sample_dim_; ++k) { pr[k] = 0.f; pi[k] = 0.f; }      // zero-padded like InputBatch::add
		labels[i] = r.label;
		current_ = (current_ + 1) % samples_.size();
	}
	return true;
}

bool MnistDataReader::Open(const std::string& image_file, const std::string& label_file, int count) {
	is_open_ = false;
	if (count <= 0) { error_ = "count must be positive"; return false; }
	std::ifstream images(image_file.c_str(), std::ios::in | std::ios::binary);
	if (images.fail()) { error_ = "Cannot open " + image_file; return false; }
	std::ifstream labels(label_file.c_str(), std::ios::in | std::ios::binary);
	if (labels.fail()) { error_ = "Cannot open " + label_file; return false; }
	images.ignore(16);                                  // magic, count, rows, columns: skipped unread, as in the reference
	labels.ignore(8);
	pixels_.resize((size_t) count * 28 * 28);
	labels_.resize((size_t) count);
	if (!images.read(reinterpret_cast<char*>(pixels_.data()), (std::streamsize) pixels_.size())) {
		error_ = image_file + " holds fewer than " + std::to_string(count) + " images"; return false;
	}
	if (!labels.read(reinterpret_cast<char*>(labels_.data()), (std::streamsize) labels_.size())) {
		error_ = label_file + " holds fewer than " + std::to_string(count) + " labels"; return false;
	}
	max_count_ = count;
	current_indx_ = 0;
	is_open_ = true;
	return true;
}

bool MnistDataReader::readData() {
	if (!is_open_) { error_ = "Open first"; return false; }
	while (current_indx_ < max_count_) {
		std::vector<std::complex<float> > sample(28 * 28);
		for (int k = 0; k < 28 * 28; ++k) {
			const float v = (float) pixels_[(size_t) current_indx_ * 28 * 28 + k];   // signed, as `char` is on the reference's platform
			sample[k] = std::complex<float>(v, v);
		}
		add(sample, (int) labels_[current_indx_]);
		++current_indx_;
	}
	return true;
}

}  // namespace cnet_b200
