// Batched data readers of the reference (data/data.h:21-165): samples held in host memory, handed out as
// InputBatch objects of the net's batch size, wrapping around at the end.  MnistDataReader reads the idx3 / idx1
// files of the MNIST distribution exactly as the reference does, quirks included: the 16- and 8-byte headers are
// skipped unread, a pixel byte is taken as a SIGNED char, and real and imaginary part are both that value
// (data/data.h:127-136).
#ifndef CNET_B200_HOST_DATA_READER_H_
#define CNET_B200_HOST_DATA_READER_H_

#include <complex>
#include <string>
#include <vector>

#include "cnet.h"

namespace cnet_b200 {

class BatchedDataReader {                               // data/data.h:30-77
	struct Record { std::vector<std::complex<float> > data; int label; };
	std::vector<Record> samples_;
	size_t current_ = 0;
protected:
	int sample_dim_;
public:
	explicit BatchedDataReader(int sample_dim) : sample_dim_(sample_dim) {}
	virtual ~BatchedDataReader() {}
	int size() const { return (int) samples_.size(); }
	int sampleDim() const { return sample_dim_; }
	void shuffle(unsigned seed);                        // the reference seeds from std::random_device; here the caller does
	bool hasNextBatch(int batch_size) const { return current_ + (size_t) batch_size <= samples_.size(); }
	InputBatch nextBatch(int batch_size);               // wraps around like the reference's
	// the same batch as split planes [batch, sample_dim] (pinned buffers for CNet::prefetchBatch) without the copy through InputBatch
	bool nextBatchInto(int batch_size, float* re, float* im, int* labels);
	void add(const std::vector<std::complex<float> >& data, int label) { samples_.push_back(Record{data, label}); }
	virtual bool readData() = 0;
};

class MnistDataReader : public BatchedDataReader {     // data/data.h:82-165
	std::vector<signed char> pixels_, labels_;
	int max_count_ = 0, current_indx_ = 0;
	bool is_open_ = false;
	std::string error_;
public:
	MnistDataReader() : BatchedDataReader(28 * 28) {}
	// reads `count` images and labels into memory; false (and error()) if a file is missing or shorter than that
	bool Open(const std::string& image_file, const std::string& label_file, int count);
	bool readData() override;                           // turns what Open read into samples
	const std::string& error() const { return error_; }
};

}  // namespace cnet_b200
#endif
