// Test infrastructure only. The reference's Configuration singleton is built on
// boost::program_options, which this image does not have. The layer sources on the LSTM
// training path read a handful of its getters; this file defines exactly those, with the
// defaults the reference's command line would give (Configuration.cpp:109-700 of the
// reference: training mode on, uniform weight init in [-0.08, 0.08], no forget-gate offset).
#include "Configuration.hpp"
#include <cstring>
Configuration *Configuration::ms_instance = NULL;
Configuration::Configuration(int, const char *[]) {
    ms_instance = this;
    m_trainingMode = true;
    m_randomSeed = 1234u;
    m_weightsDistribution = DISTRIBUTION_UNIFORM;
    m_weightsUniformMin = -0.08f;
    m_weightsUniformMax = 0.08f;
    m_weightsNormalSigma = 0.1f;
    m_weightsNormalMean = 0;
    m_lstmForgetIni = 0;
    m_auxDataDim = -1;
    m_optimizerOption = 0;
    m_seqWeightsFlag = 0;
    m_batchnorm_genmode = 0;
}
Configuration::~Configuration() {}
const Configuration &Configuration::instance() { return *ms_instance; }
bool Configuration::trainingMode() const { return m_trainingMode; }
unsigned Configuration::randomSeed() const { return m_randomSeed; }
Configuration::distribution_type_t Configuration::weightsDistributionType() const { return m_weightsDistribution; }
real_t Configuration::weightsDistributionUniformMin() const { return m_weightsUniformMin; }
real_t Configuration::weightsDistributionUniformMax() const { return m_weightsUniformMax; }
real_t Configuration::weightsDistributionNormalSigma() const { return m_weightsNormalSigma; }
real_t Configuration::weightsDistributionNormalMean() const { return m_weightsNormalMean; }
const real_t &Configuration::lstmForgetIni() const { return m_lstmForgetIni; }
const std::string &Configuration::auxillaryDataDir() const { return m_auxDataDir; }
const int &Configuration::auxillaryDataDim() const { return m_auxDataDim; }
const int &Configuration::batchnorm_genmode() const { return m_batchnorm_genmode; }
const std::string &Configuration::dataTargetPath() const { return m_dataTargetPath; }
const int &Configuration::seqWeightsFlag() const { return m_seqWeightsFlag; }
