/*
 * bkm-bucketing - the update step alone, with the flag names, defaults, units and output format of
 * the bucketing executable of krulis-martin/cuda-kmeans
 * (experimental/bucketing-cuda/bucketing-cuda/bucketing-cuda.cpp: arguments :253-278, run :161-218),
 * so that rows measured on B200 can sit beside the reference's results/updates-*.csv and
 * results/atomic-fake-*.csv:
 *
 *   bkm-bucketing --N 8M --dim 32 --k 1024 --iterations 4 --layout aos --algorithm b200 --verify
 *
 * Every iteration is an independent batch of N vectors with N bucket indices; the result of a
 * batch is the k x dim matrix of per-bucket SUMS (no sizes, no divide).  stdout:
 * "<ms per iteration> <ns per input float>"; progress messages go to stderr.
 *
 * Algorithms: serial (the default, as in the reference), b200 (automatic variant), b200_sorted,
 * b200_rows, b200_shared, b200_global (bkm_bucket_sums_f32 with that update variant), and the two
 * write-only probes b200_fake / b200_fake_shm (bkm_probe_atomics_f32).
 * Layouts: aos, soa, and the aligned aos32 / soa32 (bucketing-cuda.cpp:227-238; rows resp. columns
 * padded to a multiple of 32 floats, headers/layout_traits.hpp:15-57).  The library works on
 * unpadded layouts; the harness runs an aligned layout as the unpadded one of the padded extent
 * (aos32: dim rounded up, soa32: N and k rounded up) with the padding zeroed, which adds nothing
 * to any sum.  The inputs are the reference executable's own for the same arguments (the padding
 * draws random numbers there too, which keeps the streams aligned).  --emul, --privatizedCopies,
 * --cudaBlockSize, --cudaBlockCount and --cudaSharedMemorySize tune the reference's own kernels:
 * accepted and ignored; --itemsPerThread is honoured by the probes; --double is refused.
 */
#include "bkm.h"
#include "reference_data.hpp"

#include <cuda_runtime.h>

#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <iostream>
#include <stdexcept>
#include <string>
#include <vector>

namespace {

struct Options {
	uint64_t n = 10240;
	uint32_t k = 512, dim = 20, iterations = 1, seed = 42, items_per_thread = 1;
	bool verify = false, dry_run = false;
	std::string algorithm = "serial", layout = "aos", out;
};

[[noreturn]] void usage_error(const std::string& what)
{
	std::cout << "Invalid arguments: " << what << std::endl << std::endl
		<< "Usage: bkm-bucketing [--N n] [--k k] [--dim d] [--iterations i] [--seed s] [--layout aos|soa|aos32|soa32]\n"
		<< "                     [--algorithm serial|b200|b200_sorted|b200_rows|b200_shared|b200_global|b200_fake|b200_fake_shm]\n"
		<< "                     [--itemsPerThread t] [--verify] [--out file] [--dryRun]\n"
		<< "Integers take the suffixes k, M, G (powers of 1024)." << std::endl;
	std::exit(1);
}

uint64_t parse_int(const std::string& name, const std::string& text)
{
	if (text.empty()) usage_error("--" + name + " needs a value");
	size_t pos = 0;
	unsigned long long v = 0;
	try { v = std::stoull(text, &pos); } catch (...) { usage_error("--" + name + ": '" + text + "' is not a number"); }
	uint64_t mult = 1;
	if (pos < text.size()) {
		const std::string suffix = text.substr(pos);
		if (suffix == "k") mult = 1024ull;
		else if (suffix == "M") mult = 1024ull * 1024;
		else if (suffix == "G") mult = 1024ull * 1024 * 1024;
		else usage_error("--" + name + ": unknown suffix '" + suffix + "'");
	}
	return (uint64_t)v * mult;
}

Options parse(int argc, char** argv)
{
	Options o;
	for (int i = 1; i < argc; ++i) {
		std::string a = argv[i];
		if (a.rfind("--", 0) != 0) usage_error("unexpected argument '" + a + "'");
		a = a.substr(2);
		auto value = [&]() -> std::string {
			if (i + 1 >= argc) usage_error("--" + a + " needs a value");
			return argv[++i];
		};
		if (a == "N") o.n = parse_int(a, value());
		else if (a == "k") o.k = (uint32_t)parse_int(a, value());
		else if (a == "dim") o.dim = (uint32_t)parse_int(a, value());
		else if (a == "iterations") o.iterations = (uint32_t)parse_int(a, value());
		else if (a == "seed") o.seed = (uint32_t)parse_int(a, value());
		else if (a == "itemsPerThread") o.items_per_thread = (uint32_t)parse_int(a, value());
		else if (a == "verify") o.verify = true;
		else if (a == "dryRun") o.dry_run = true;
		else if (a == "emul") {}
		else if (a == "algorithm") o.algorithm = value();
		else if (a == "layout") o.layout = value();
		else if (a == "out") o.out = value();
		else if (a == "cudaBlockSize" || a == "cudaBlockCount" || a == "cudaSharedMemorySize" || a == "privatizedCopies") (void)value();
		else if (a == "double") usage_error("--double: the B200 kernels are fp32 only");
		else usage_error("unknown argument '--" + a + "'");
	}
	// the reference's lower bounds (bucketing-cuda.cpp:253-257)
	if (o.dim < 2 || o.k < 2 || o.n < 128 || o.iterations < 1 || o.items_per_thread < 1)
		usage_error("dim >= 2, k >= 2, N >= 128, iterations >= 1 and itemsPerThread >= 1 are required");
	if (o.layout != "aos" && o.layout != "soa" && o.layout != "aos32" && o.layout != "soa32") usage_error("layout must be aos, soa, aos32 or soa32");
	return o;
}

// Geometry of one layout (headers/layout_traits.hpp:15-57): element (item, d) of `items` vectors.
struct Layout {
	bool soa;
	uint32_t align;
	size_t stride(size_t items, size_t dim) const { return soa ? (items + align - 1) / align * align : (dim + align - 1) / align * align; }
	size_t size(size_t items, size_t dim) const { return soa ? stride(items, dim) * dim : stride(items, dim) * items; }
	size_t at(size_t item, size_t d, size_t items, size_t dim) const { return soa ? d * stride(items, dim) + item : item * stride(items, dim) + d; }
};

void check(int rc)
{
	if (rc != BKM_OK) throw std::runtime_error(bkm_last_error());
}

void cuda_ok(cudaError_t e, const char* what)
{
	if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

double now_ms()
{
	return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

// The reference's acceptance rule for this step (bucketing-cuda.cpp:105-142): relative error
// |a-b| / max(|a|+|b|, 5e-5) <= 5e-5 for every value.
bool verify(const std::vector<float>& res, const std::vector<float>& want, size_t dim, size_t k, double tol = 0.00005)
{
	if (res.size() != want.size()) {
		std::cerr << std::endl << "Error: Result size mismatch (" << res.size() << " values found, but " << want.size() << " values expected)!" << std::endl;
		return false;
	}
	size_t errors = 0;
	for (size_t i = 0; i < res.size(); ++i) {
		const double a = res[i], b = want[i];
		const double err = std::fabs(a - b) / std::max(std::fabs(a) + std::fabs(b), tol);
		if (!(err <= tol)) {
			if (errors == 0) std::cerr << std::endl;
			if (++errors <= 10)
				std::cerr << "Error at iteration #" << (i / dim) / k << " [" << (i / dim) % k << "][" << (i % dim) << "]: " << res[i] << " != " << want[i] << std::endl;
		}
	}
	if (errors) std::cerr << "Total errors found: " << errors << std::endl;
	return errors == 0;
}

int run(const Options& o)
{
	int variant = -1;
	bool fake = false, fake_shm = false;
	if (o.algorithm == "b200") variant = BKM_UPDATE_AUTO;
	else if (o.algorithm == "b200_sorted") variant = BKM_UPDATE_SORTED;
	else if (o.algorithm == "b200_rows") variant = BKM_UPDATE_ROWS;
	else if (o.algorithm == "b200_shared") variant = BKM_UPDATE_SHARED;
	else if (o.algorithm == "b200_global") variant = BKM_UPDATE_GLOBAL;
	else if (o.algorithm == "b200_fake") fake = true;
	else if (o.algorithm == "b200_fake_shm") fake = fake_shm = true;
	else if (o.algorithm != "serial") throw std::runtime_error("Unkown algorithm '" + o.algorithm + "'.");
	const Layout lay{o.layout == "soa" || o.layout == "soa32", (o.layout == "aos32" || o.layout == "soa32") ? 32u : 1u};
	if (o.dry_run) {
		std::cout << "N=" << o.n << " k=" << o.k << " dim=" << o.dim << " iterations=" << o.iterations << " seed=" << o.seed
			<< " layout=" << o.layout << " algorithm=" << o.algorithm << " itemsPerThread=" << o.items_per_thread << " verify=" << o.verify << std::endl;
		return 0;
	}

	const size_t n = o.n, k = o.k, dim = o.dim, iters = o.iterations;
	const size_t data_size = lay.size(n, dim), res_size = lay.size(k, dim);
	std::cerr << "Generating input data (" << n << " x " << dim << "), " << iters << " iterations ..." << std::endl;
	std::cerr << "Seed is set to " << o.seed << std::endl;
	std::vector<float> data(data_size * iters);
	std::vector<uint32_t> indices(n * iters);
	refdata::bucketing_inputs(data, indices, o.k, o.seed);
	std::cerr << "Selected algorithm: " << o.algorithm << std::endl;

	// serial sums in point order, as the reference's SerialBucketingAlgorithm (headers/serial.hpp:36-58);
	// results are reported per iteration as k rows of dim values without padding (:61-79)
	auto serial = [&](std::vector<float>& out) {
		out.assign(k * dim * iters, 0.0f);
		for (size_t it = 0; it < iters; ++it)
			for (size_t i = 0; i < n; ++i) {
				const size_t target = indices[it * n + i];
				for (size_t d = 0; d < dim; ++d) out[(it * k + target) * dim + d] += data[it * data_size + lay.at(i, d, n, dim)];
			}
	};

	std::vector<float> result;
	double init_ms = 0.0, run_ms = 0.0;
	if (o.algorithm == "serial") {
		std::cerr << "Initializing ... 0 ms" << std::endl;
		std::cerr << "Running ... ";
		const double t0 = now_ms();
		serial(result);
		run_ms = now_ms() - t0;
	} else {
		// the library's (unpadded) view of the buffers: an aligned layout is the plain one of the padded extent
		const size_t lib_n = lay.soa ? lay.stride(n, dim) : n;
		const size_t lib_k = lay.soa ? lay.stride(k, dim) : k;
		const size_t lib_dim = lay.soa ? dim : lay.stride(n, dim);
		std::cerr << "Initializing ... ";
		double t0 = now_ms();
		std::vector<float*> d_data(iters, nullptr), d_res(iters, nullptr);
		std::vector<uint32_t*> d_idx(iters, nullptr);
		void* ws = nullptr;
		const size_t ws_bytes = bkm_workspace_bytes(lib_n, (uint32_t)lib_k, (uint32_t)lib_dim);
		if (ws_bytes == 0) throw std::runtime_error("problem size not supported");
		cuda_ok(cudaMalloc(&ws, ws_bytes), "cudaMalloc");
		std::vector<float> clean(data_size);
		std::vector<uint32_t> idx(lib_n, 0u);
		for (size_t it = 0; it < iters; ++it) {
			cuda_ok(cudaMalloc(&d_data[it], data_size * sizeof(float)), "cudaMalloc");
			cuda_ok(cudaMalloc(&d_res[it], res_size * sizeof(float)), "cudaMalloc");
			cuda_ok(cudaMalloc(&d_idx[it], lib_n * sizeof(uint32_t)), "cudaMalloc");
			// padding elements are zeroed (they would be added into the sums of the padded extent)
			std::fill(clean.begin(), clean.end(), 0.0f);
			for (size_t i = 0; i < n; ++i)
				for (size_t d = 0; d < dim; ++d) clean[lay.at(i, d, n, dim)] = data[it * data_size + lay.at(i, d, n, dim)];
			std::copy(indices.begin() + it * n, indices.begin() + (it + 1) * n, idx.begin());
			cuda_ok(cudaMemcpy(d_data[it], clean.data(), data_size * sizeof(float), cudaMemcpyHostToDevice), "copy");
			cuda_ok(cudaMemcpy(d_idx[it], idx.data(), lib_n * sizeof(uint32_t), cudaMemcpyHostToDevice), "copy");
			cuda_ok(cudaMemset(d_res[it], 0, res_size * sizeof(float)), "memset");
		}
		cuda_ok(cudaDeviceSynchronize(), "sync");
		init_ms = now_ms() - t0;
		std::cerr << init_ms << " ms" << std::endl;
		std::cerr << "Running ... ";
		t0 = now_ms();
		for (size_t it = 0; it < iters; ++it) {
			if (fake) check(bkm_probe_atomics_f32(d_res[it], lib_n, (uint32_t)lib_k, (uint32_t)lib_dim, lay.soa, fake_shm, o.items_per_thread, nullptr));
			else check(bkm_bucket_sums_f32(d_data[it], d_idx[it], d_res[it], lib_n, (uint32_t)lib_k, (uint32_t)lib_dim, lay.soa, variant, ws, ws_bytes, nullptr));
		}
		cuda_ok(cudaDeviceSynchronize(), "CUDA error after the run");
		run_ms = now_ms() - t0;
		if (!fake) check(bkm_workspace_check(ws, nullptr));
		std::vector<float> tmp(res_size);
		result.reserve(k * dim * iters);
		for (size_t it = 0; it < iters; ++it) {
			cuda_ok(cudaMemcpy(tmp.data(), d_res[it], res_size * sizeof(float), cudaMemcpyDeviceToHost), "copy back");
			for (size_t c = 0; c < k; ++c)
				for (size_t d = 0; d < dim; ++d) result.push_back(tmp[lay.at(c, d, k, dim)]);
			cudaFree(d_data[it]); cudaFree(d_res[it]); cudaFree(d_idx[it]);
		}
		cudaFree(ws);
	}

	std::cout << run_ms / (double)iters;
	std::cerr << " ms/iter (which is";
	std::cout << " " << (run_ms * 1000000.0 / ((double)iters * dim * (double)n));
	std::cerr << " ns/input float)";
	std::cout << std::endl;

	int rc = 0;
	if (o.verify) {
		std::cerr << "Verifying results ... ";
		std::vector<float> want;
		if (fake) {
			// what the probe writes: 0.1 per value landing in bucket (i / dim) % k over the library's extent
			want.assign(k * dim * iters, 0.0f);
			const size_t lib_n = lay.soa ? lay.stride(n, dim) : n, lib_k = lay.soa ? lay.stride(k, dim) : k, lib_dim = lay.soa ? dim : lay.stride(n, dim);
			std::vector<double> one(lib_k * lib_dim, 0.0);
			for (size_t i = 0; i < lib_n * lib_dim; ++i) one[((i / lib_dim) % lib_k) * lib_dim + i % lib_dim] += 1.0;
			for (size_t it = 0; it < iters; ++it)
				for (size_t c = 0; c < k; ++c)
					for (size_t d = 0; d < dim; ++d) want[(it * k + c) * dim + d] = (float)(0.1 * one[c * lib_dim + d]);
		} else {
			serial(want);
		}
		// the probes add one constant thousands of times into one float: its rounding accumulates, so
		// their check is a sanity check of the bucket pattern with a wider band
		if (verify(result, want, dim, k, fake ? 0.002 : 0.00005)) std::cerr << "OK" << std::endl;
		else { std::cerr << "FAILED" << std::endl; rc = 3; }
	}
	if (!o.out.empty()) {
		std::cerr << "Saving results to " << o.out << " ..." << std::endl;
		FILE* f = std::fopen(o.out.c_str(), "w");
		if (!f) throw std::runtime_error("cannot open '" + o.out + "' for writing");
		for (size_t i = 0; i < result.size();) {
			for (size_t d = 0; d < dim; ++d) std::fprintf(f, d ? "\t%g" : "%g", result[i++]);
			std::fprintf(f, "\n");
		}
		std::fclose(f);
	}
	std::cerr << "And we're done here." << std::endl;
	return rc;
}

} // namespace

int main(int argc, char** argv)
{
	const Options o = parse(argc, argv);
	try {
		return run(o);
	} catch (std::exception& e) {
		std::cout << "Error: " << e.what() << std::endl << std::endl;
		return 2;
	}
}
